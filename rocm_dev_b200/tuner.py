"""Grid-search tuner for the skinny FP8 GEMM, in the spirit of the reference's
``grid.py`` (grid.py:40-145 in the reference project).

The reference tunes by rewriting ``#define``s in ``core.cu`` and recompiling
each candidate under a 100 s timeout; here the knobs (tile rows, K split,
ring stages) are run-time arguments of ``rdb_skinny_gemm_fp8_tuned``, every
device-side wait is bounded, and a candidate is one CUDA-graph timing.  Results
are appended to a JSON-lines file so that an interrupted search can be resumed
(``--restart N`` skips the first N candidates, as grid.py:72-73 does).

    python -m rocm_dev_b200.tuner -a "8 4096 4096" [-s] [-r N] [-o results.jsonl] [--table tuned.txt]
    python -m rocm_dev_b200.tuner -p dense -a "4096 4096 4096" --table tuned.txt

With ``--table`` the winner is written into a tuning-table file (one line per
shape, rewritten in place) when it beats the automatic plan; the launchers
load that file through ``rdb_tuning_table_load`` or the environment variable
``RDB_TUNING_TABLE`` - the counterpart of the reference compiling the chosen
``#define``s in (grid.py:106-116).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os

MAX_CLUSTERS = [0, 148, 74, 45, 33, 26, 22, 15, 15]      # resident clusters per size on a 148-SM part


def candidates(M: int, N: int, K: int, max_clusters=MAX_CLUSTERS, stages=(2, 3, 4, 6, 8)):
    """(rows_per_tile, split_k, stages) triples worth timing: tiles that fit one
    wave, at least 64 CTAs, a ring of at most ~200 KiB."""
    mpad = 16 if M <= 16 else 32
    num_kb = (K + 127) // 128
    out = []
    for sk in range(1, 9):
        if sk > num_kb:
            break
        rows = set()
        for T in range((N + 255) // 256, max_clusters[sk] + 1):
            r = ((N + T - 1) // T + 15) // 16 * 16
            if r <= 256:
                rows.add(r)
        for r in sorted(rows, reverse=True):
            ctas = ((N + r - 1) // r) * sk
            if ctas < min(64, ((N + 15) // 16) * sk):
                continue
            kb_per = (num_kb + sk - 1) // sk
            for st in stages:
                if st > kb_per or st * (mpad + r) * 128 > 200 * 1024:
                    continue
                out.append((r, sk, st))
    return out


def automatic_plan(M: int, N: int, K: int, sm_count: int = 148):
    from ._lib import lib
    r, s, st = C.c_int(), C.c_int(), C.c_int()
    lib().rdb_skinny_gemm_plan(M, N, K, sm_count, C.byref(r), C.byref(s), C.byref(st))
    return r.value, s.value, st.value


def time_config(M, N, K, rows, split_k, stages, flags=1, iters=30, copies=None):
    """Mean microseconds per launch of one configuration (CUDA graph replay,
    weight copies rotating so that reads stay L2-cold)."""
    import torch

    from . import skinny_gemm_fp8_tuned
    from ._lib import lib
    dev = torch.device("cuda")
    key = (N, K)
    cache = time_config.__dict__.setdefault("cache", {})
    if key not in cache:
        cache.clear()
        n = copies or max(2, int(400e6 // (N * K)) + 1)
        cache[key] = [torch.randint(0, 0x7E, (N, K), dtype=torch.uint8, device=dev) for _ in range(n)]
    Bs = cache[key]
    A = torch.randint(0, 0x7E, (M, K), dtype=torch.uint8, device=dev)
    one = torch.ones(1, device=dev)
    D = torch.empty((M, N), dtype=torch.bfloat16, device=dev)

    def call(i):
        code = skinny_gemm_fp8_tuned(A, Bs[i % len(Bs)], one, one, D, rows, split_k, stages, flags)
        if code != 0:
            raise RuntimeError(f"status {code}")
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for i in range(2):
            call(i)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            for i in range(iters):
                call(i)
        g.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(3):
            g.replay()
        b.record(stream)
        torch.cuda.synchronize()
    if lib().rdb_device_status() != 0:
        raise RuntimeError("device-side wait timed out")
    return a.elapsed_time(b) * 1e3 / (3 * iters)


def read_table(path: str) -> dict:
    """{("skinny", mpad, N, K): (rows, split_k, stages), ("dense", M, N, K): (tile_rows, max_ctas)}"""
    table = {}
    if os.path.exists(path):
        for line in open(path):
            f = line.split("#")[0].split()
            if f:
                table[(f[0], int(f[1]), int(f[2]), int(f[3]))] = tuple(int(x) for x in f[4:])
    return table


def write_table(path: str, table: dict) -> None:
    lines = ["# tuning table of rocm_dev_b200: measured best configurations, loaded with rdb_tuning_table_load",
             "# skinny <m_bucket> <N> <K> <rows_per_tile> <split_k> <stages> | dense <M> <N> <K> <tile_rows> <max_ctas>"]
    for key in sorted(table):
        lines.append(" ".join(str(x) for x in (*key, *table[key])))
    tmp = path + ".tmp"
    with open(tmp, "w") as f:
        f.write("\n".join(lines) + "\n")
    os.replace(tmp, path)


def dense_candidates(M: int, N: int, K: int, sm_count: int = 148):
    """(tile_rows, max_ctas) pairs: the three tilings (CTA pairs need K % 128 == 0)
    on the whole machine and on slightly fewer CTAs (a tile count that does not
    divide by the SM count can finish sooner on a grid that divides it)."""
    out = []
    for tr in (2, 3, 256, 128):
        if tr in (2, 3) and K % 128:
            continue
        rows = 128 if tr == 128 else 256
        tiles = -(-M // rows) * -(-N // 256)
        unit = 2 if tr in (2, 3) else 1
        grids = {0}
        for waves in range(1, 9):
            g = -(-tiles // waves)
            g += g % unit
            if sm_count // 2 <= g < sm_count:
                grids.add(g)
        out += [(tr, g) for g in sorted(grids)]
    return out


def time_dense(M, N, K, tile_rows, max_ctas, iters=10):
    import torch

    from . import dense_gemm_fp8
    from ._lib import lib
    dev = torch.device("cuda")
    A = torch.randint(0, 0x78, (M, K), dtype=torch.uint8, device=dev)
    B = torch.randint(0, 0x78, (N, K), dtype=torch.uint8, device=dev)
    D = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    one = torch.ones(1, device=dev)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for _ in range(2):
            dense_gemm_fp8(A, B, one, one, out=D, tile_rows=tile_rows, max_ctas=max_ctas)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(iters):
            dense_gemm_fp8(A, B, one, one, out=D, tile_rows=tile_rows, max_ctas=max_ctas)
        b.record(stream)
        torch.cuda.synchronize()
    if lib().rdb_device_status() != 0:
        raise RuntimeError("device-side wait timed out")
    return a.elapsed_time(b) * 1e3 / iters


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--project", "-p", default="skinny_gemm", choices=["skinny_gemm", "dense"])
    ap.add_argument("--table", default="", help="tuning-table file to update with the winner")
    ap.add_argument("--arguments", "-a", required=True, help='"m n k"')
    ap.add_argument("--restart", "-r", type=int, default=0, help="skip the first N candidates")
    ap.add_argument("--shuffle", "-s", action="store_true")
    ap.add_argument("--output", "-o", default="")
    a = ap.parse_args(argv)
    M, N, K = (int(x) for x in a.arguments.split())
    if a.project == "dense":
        return main_dense(a, M, N, K)
    from ._lib import lib
    lib().rdb_tuning_table_clear()           # time the analytic plan, not an earlier table entry
    cands = candidates(M, N, K)
    if a.shuffle:
        import random
        random.Random(0).shuffle(cands)
    out_path = a.output or f"tune_{M}_{N}_{K}.jsonl"
    auto = automatic_plan(M, N, K)
    best = None
    for idx, (r, sk, st) in enumerate(cands):
        if idx < a.restart:
            continue
        try:
            us = time_config(M, N, K, r, sk, st)
        except RuntimeError as e:          # a bad candidate reports an error instead of hanging
            us = None
            err = str(e)
        rec = {"index": idx, "rows": r, "split_k": sk, "stages": st, "us": us}
        if us is None:
            rec["error"] = err
        with open(out_path, "a") as f:
            f.write(json.dumps(rec) + "\n")
        if us is not None and (best is None or us < best["us"]):
            best = rec
    auto_us = time_config(M, N, K, 0, 0, 0)
    by = N * K + M * K + 2 * M * N + 8
    summary = {"shape": [M, N, K], "candidates": len(cands), "best": best, "automatic_plan": list(auto),
               "automatic_us": auto_us, "best_gbs": by / best["us"] / 1e3 if best else None,
               "automatic_gbs": by / auto_us / 1e3, "results": os.path.abspath(out_path)}
    if a.table and best and best["us"] < auto_us:
        table = read_table(a.table)
        table[("skinny", 16 if M <= 16 else 32, N, K)] = (best["rows"], best["split_k"], best["stages"])
        write_table(a.table, table)
        summary["table"] = os.path.abspath(a.table)
    print(json.dumps(summary))
    return summary


def main_dense(a, M, N, K):
    from ._lib import lib
    lib().rdb_tuning_table_clear()
    out_path = a.output or f"tune_dense_{M}_{N}_{K}.jsonl"
    best = None
    cands = dense_candidates(M, N, K)
    for idx, (tr, mc) in enumerate(cands):
        if idx < a.restart:
            continue
        try:
            us, err = time_dense(M, N, K, tr, mc), None
        except Exception as e:  # noqa: BLE001  (a refused configuration reports an error instead of hanging)
            us, err = None, str(e)
        rec = {"index": idx, "tile_rows": tr, "max_ctas": mc, "us": us}
        if err:
            rec["error"] = err
        with open(out_path, "a") as f:
            f.write(json.dumps(rec) + "\n")
        if us is not None and (best is None or us < best["us"]):
            best = rec
    auto_us = time_dense(M, N, K, 0, 0)
    summary = {"project": "dense", "shape": [M, N, K], "candidates": len(cands), "best": best, "automatic_us": auto_us,
               "best_tflops": 2.0 * M * N * K / best["us"] / 1e6 if best else None,
               "automatic_tflops": 2.0 * M * N * K / auto_us / 1e6, "results": os.path.abspath(out_path)}
    if a.table and best and best["us"] < auto_us:
        table = read_table(a.table)
        table[("dense", M, N, K)] = (best["tile_rows"], best["max_ctas"])
        write_table(a.table, table)
        summary["table"] = os.path.abspath(a.table)
    print(json.dumps(summary))
    return summary


if __name__ == "__main__":
    main()
