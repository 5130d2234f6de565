#!/usr/bin/env python
"""Benchmark of the hot path: the skinny FP8 GEMM decode sweep.

One "step" is one decode pass over the four Llama-3-8B-shaped projections
(QKV 6144x4096, O 4096x4096, gate_up 28672x4096, down 4096x14336) at each
M in {1, 2, 4, 8, 16}: 20 launches of the skinny FP8 GEMM on synthetic e4m3
operands.  `value` is the algorithmic HBM traffic of those launches
(N*K + M*K + 2*M*N + 8 bytes each) divided by the device time, in GB/s, summed
over ranks (the path does not shard: N > 1 runs independent replicas).

    python bench.py --gpus N --steps K --warmup W [--impl reference]

With --impl reference the CPU restatement of the reference's host GEMM (the
oracle port; the reference's own HIP sources cannot be compiled here) is timed
on the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPES = [("qkv", 6144, 4096), ("o", 4096, 4096), ("gate_up", 28672, 4096), ("down", 4096, 14336)]
MS = [1, 2, 4, 8, 16]
WEIGHT_SETS = 2
# DRAM bytes (read + write) per algorithmic byte from the ncu capture summarised in
# profiles/skinny_gemm_gate_up_M8_full.md (121.5 MB moved for 117.9 MB algorithmic); traffic scales with the bytes.
TRAFFIC_PER_ALGO_BYTE = 1.03
METRIC = "skinny FP8 GEMM HBM GB/s, decode sweep M=1..16 over Llama-3-8B-shaped (N,K)"


def algo_bytes(M, N, K):
    return N * K + M * K + 2 * M * N + 8


def step_bytes():
    return sum(algo_bytes(M, N, K) for M in MS for _, N, K in SHAPES)


def measured_peak():
    """HBM peak in GB/s: the driver-written measurement, else the fallback."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons (read-only NVML queries) every
    10 ms on a thread while a region runs."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index):
        self.index, self.sm, self.mask, self.max_mhz = index, [], 0, None
        self._stop = threading.Event()
        self._thread = None
        self.error = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            idx = self.index
            if visible:
                ent = visible.split(",")[self.index]
                idx = int(ent) if ent.isdigit() else self.index
            h = pynvml.nvmlDeviceGetHandleByIndex(idx)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))

            def loop():
                while not self._stop.is_set():
                    try:
                        self.sm.append(float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)))
                        self.mask |= int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(h))
                    except Exception as e:  # noqa: BLE001
                        self.error = str(e)
                        return
                    time.sleep(0.01)
            self._thread = threading.Thread(target=loop, daemon=True)
            self._thread.start()
        except Exception as e:  # noqa: BLE001
            self.error = str(e)

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=1.0)
        sm = sorted(self.sm)
        reasons = [n for bit, n in self.REASONS.items() if self.mask & bit]
        out = {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(reasons),
               "samples": len(sm)}
        if self.error:
            out["error"] = self.error
        return out


# ------------------------------------------------------------------ CPU arm
class CpuWorkload:
    """The decode sweep on the host: the oracle's sequential-fp32 GEMM (the
    restatement of the reference's host loop) over the same 20 (shape, M)
    cases, rows spread over all host threads.  Operands are generated once."""

    def __init__(self, ms=MS):
        import numpy as np
        from oracle import oracle as O
        O.build()
        self.O, self.ms = O, list(ms)
        rng = np.random.default_rng(0)
        self.B = [rng.integers(0, 0x7E, (N, K), dtype=np.uint8) for _, N, K in SHAPES]
        self.A = {(M, K): rng.integers(0, 0x7E, (M, K), dtype=np.uint8) for M in self.ms
                  for K in {k for _, _, k in SHAPES}}
        self.bytes = sum(algo_bytes(M, N, K) for M in self.ms for _, N, K in SHAPES)
        self.threads = O.num_threads()

    def step(self):
        t0 = time.perf_counter()
        for M in self.ms:
            for si, (_, N, K) in enumerate(SHAPES):
                self.O.gemm_fp8_bf16(self.A[(M, K)], self.B[si], 0.01, 0.001)
        return time.perf_counter() - t0


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w = CpuWorkload()
    for _ in range(min(args.warmup, 2)):
        w.step()
    probe = w.step()
    # bounded: at most ~90 s of CPU work however many steps were asked for
    steps = max(1, min(args.steps, int(90.0 / max(probe, 1e-3))))
    dt = sum(w.step() for _ in range(steps))
    v = w.bytes * steps / dt / 1e9
    sample = (f"{steps} step(s) of the full sweep (20 GEMMs, M in {MS}) with the sequential-fp32 host GEMM on "
              f"{w.threads} threads")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": "GB/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": min(args.warmup, 2), "ms_per_step": dt / steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp8_e4m3 x fp8_e4m3 -> f32", "data": "synthetic",
        "config": {"workload": "configs[1]: decode sweep M in {1,2,4,8,16} x {qkv,o,gate_up,down}",
                   "shapes": [[n, k] for _, n, k in SHAPES], "M": MS},
        "cpu_baseline": {"value": v, "unit": "GB/s", "cores": w.threads, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ------------------------------------------------------------------ GPU arm
def run_gpu(args):
    import torch
    import torch.distributed as dist

    import rocm_dev_b200 as R
    from rocm_dev_b200 import quant

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    R.lib()
    if world > 1:
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")   # keep stdout for the one JSON line
        dist.init_process_group("nccl", device_id=dev)

    # synthetic operands with the value distribution of quantised N(0,1) / N(0,0.02)
    weights = []
    for s in range(WEIGHT_SETS):
        weights.append([quant.synthetic_weights_fast(N, K, seed=100 * s + i, device=dev) for i, (_, N, K) in
                        enumerate(SHAPES)])
    acts = {}
    for M in MS:
        for K in sorted({k for _, _, k in SHAPES}):
            g = torch.Generator(device=dev).manual_seed(M * 131 + K)
            a = torch.randn((M, K), generator=g, device=dev)
            amax = a.abs().max()
            acts[(M, K)] = ((a * (448.0 / amax)).to(torch.float8_e4m3fn).view(torch.uint8), (amax / 448.0).reshape(1))
    outs = {(M, N): torch.empty((M, N), dtype=torch.bfloat16, device=dev) for M in MS for _, N, _ in SHAPES}

    flags = R.OVERLAP_PRIOR_KERNEL   # weights are never written inside the timed region

    if args.single and not args.single.split("_M")[0] in [n for n, _, _ in SHAPES]:
        return run_single_other(args, torch, R, quant, dev)
    if args.single:
        # profiling aid: plain launches of one (shape, M) case, weight copies rotating
        name, m = args.single.rsplit("_M", 1)
        si = [n for n, _, _ in SHAPES].index(name)
        M, (_, N, K) = int(m), SHAPES[si]
        Aq, sa = acts[(M, K)]
        for i in range(args.warmup + args.steps):
            Bq, sb = weights[i % WEIGHT_SETS][si]
            R.skinny_gemm_fp8_tuned(Aq, Bq, sa, sb, outs[(M, N)], 0, 0, 0, 0)
        torch.cuda.synchronize()
        print(json.dumps({"single": args.single, "launches": args.warmup + args.steps,
                          "algorithmic_bytes_per_launch": algo_bytes(M, N, K)}))
        return

    def one_step(step_idx):
        n = 0
        for mi, M in enumerate(MS):
            wset = weights[(step_idx * len(MS) + mi) % WEIGHT_SETS]
            for si, (_, N, K) in enumerate(SHAPES):
                Aq, sa = acts[(M, K)]
                Bq, sb = wset[si]
                code = R.skinny_gemm_fp8_tuned(Aq, Bq, sa, sb, outs[(M, N)], 0, 0, 0, flags)
                if code != 0:
                    raise RuntimeError(f"skinny GEMM returned {code}")
                n += 1
        return n

    stream = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(stream):
        launches_per_step = one_step(0)
        torch.cuda.synchronize()
        # two graphs (even / odd step) so that the weight sets keep alternating
        graphs = []
        for parity in range(2):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                one_step(parity)
            graphs.append(g)
        for w in range(max(args.warmup, 3)):
            graphs[w % 2].replay()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.profiler.start()          # lets `ncu --profile-from-start off` see only the timed region
        e0.record(stream)
        for s in range(args.steps):
            graphs[s % 2].replay()
        e1.record(stream)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        if world > 1:
            dist.barrier()
        clocks = sampler.stop() if rank == 0 else None
        ms = e0.elapsed_time(e1)
    if R.lib().rdb_device_status() != 0:
        raise RuntimeError("device status word reports a timed-out wait")
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())

    # per-shape detail (rank 0): each (shape, M) alone, rotating weight copies > L2
    detail = {}
    if rank == 0 and not args.no_detail:
        with torch.cuda.stream(stream):
            for si, (name, N, K) in enumerate(SHAPES):
                copies = [weights[s][si] for s in range(WEIGHT_SETS)]
                while sum(c[0].numel() for c in copies) < 300e6:
                    copies.append(quant.synthetic_weights_fast(N, K, seed=977 + len(copies), device=dev))
                for M in MS:
                    Aq, sa = acts[(M, K)]
                    g = torch.cuda.CUDAGraph()
                    iters = 24
                    for i in range(2):
                        R.skinny_gemm_fp8_tuned(Aq, copies[i % len(copies)][0], sa, copies[0][1], outs[(M, N)], 0, 0, 0, flags)
                    torch.cuda.synchronize()
                    with torch.cuda.graph(g, stream=stream):
                        for i in range(iters):
                            R.skinny_gemm_fp8_tuned(Aq, copies[i % len(copies)][0], sa, copies[0][1], outs[(M, N)], 0, 0,
                                                    0, flags)
                    g.replay()
                    torch.cuda.synchronize()
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record(stream)
                    for _ in range(3):
                        g.replay()
                    b.record(stream)
                    torch.cuda.synchronize()
                    us = a.elapsed_time(b) * 1e3 / (3 * iters)
                    detail[f"{name}_M{M}"] = {"us": round(us, 2), "gbs": round(algo_bytes(M, N, K) / us / 1e3, 1)}
                del copies

    # end to end through the host-buffer entry: every operand H2D, result D2H, each call
    e2e = None
    if not args.no_e2e:
        host_w = [(w[0].cpu().pin_memory(), w[1].cpu().pin_memory()) for w in weights[0]]
        host_a = {k: (v[0].cpu().pin_memory(), v[1].cpu().pin_memory()) for k, v in acts.items()}
        host_o = {k: torch.empty(v.shape, dtype=torch.bfloat16).pin_memory() for k, v in outs.items()}
        h2d = sum(N * K + 4 + M * K + 4 for M in MS for _, N, K in SHAPES)
        d2h = sum(2 * M * N for M in MS for _, N, _ in SHAPES)

        def e2e_step():
            for M in MS:
                for si, (_, N, K) in enumerate(SHAPES):
                    R.skinny_gemm_fp8_host(host_a[(M, K)][0], host_w[si][0], host_a[(M, K)][1], host_w[si][1],
                                           host_o[(M, N)], device=dev)
        e2e_step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        n_e2e = max(2, min(args.steps, 4))
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n_e2e):
            e2e_step()
        b.record()
        torch.cuda.synchronize()
        e2e_ms = a.elapsed_time(b)
        if world > 1:
            t = torch.tensor([e2e_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = float(t.item())
        e2e = {"value": world * step_bytes() * n_e2e / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": n_e2e,
               "note": "weights, activations and scales copied from pinned host memory for every call"}

    allreduce = None
    if world > 1 and not args.no_allreduce:
        allreduce = bench_allreduce(torch, dist, R, dev, rank, world)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    total_bytes = world * step_bytes() * args.steps
    value = total_bytes / (ms * 1e-3) / 1e9
    peak, peak_kind = measured_peak()
    per_gpu = value / world
    cpu = None
    if world == 1 and not args.no_cpu:
        w = CpuWorkload()
        w.step()
        reps = 3
        dt = sum(w.step() for _ in range(reps))
        cpu = {"value": w.bytes * reps / dt / 1e9, "unit": "GB/s", "cores": w.threads, "kind": "port",
               "sample": f"{reps} steps of the full sweep with the oracle's sequential-fp32 GEMM ({dt:.1f} s)"}
    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp8_e4m3 x fp8_e4m3 -> f32", "data": "synthetic",
        "config": {"workload": "configs[1]: decode sweep M in {1,2,4,8,16} x {qkv,o,gate_up,down}",
                   "shapes": [[n, k] for _, n, k in SHAPES], "M": MS, "launches_per_step": launches_per_step,
                   "l2": f"inputs larger than L2: {WEIGHT_SETS} weight sets of 218 MB alternate, a matrix is re-read "
                         "only after 436 MB of other weights", "launch": "CUDA graph, programmatic dependent launch",
                   "multi_gpu": "replicas only"},
        "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s", "frac": per_gpu / peak,
                     "traffic": TRAFFIC_PER_ALGO_BYTE * step_bytes() / launches_per_step, "peak_kind": f"of {peak_kind}", "kernel": "skinny_gemm_kernel",
                     "algorithmic_bytes_per_launch": step_bytes() / launches_per_step,
                     "avg_launch_us": ms * 1e3 / (args.steps * launches_per_step)},
        "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches_per_step * args.steps, "clocks": clocks,
        "detail": detail,
    }
    if allreduce is not None:
        line["allreduce"] = allreduce
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def bench_allreduce(torch, dist, R, dev, rank, world):
    """FP8-encoded allreduce against NCCL's bf16 allreduce on [T, 8192] bf16
    tensors.  busBW = S/t * 2(n-1)/n with S the bf16 size; device time, max over
    ranks.  Reported beside the headline metric when more than one GPU runs."""
    ar = R.Fp8AllReduce(max_elems=4096 * 8192, backend="auto")
    out = {"unit": "GB/s busBW", "world": world, "workspace": ar.backend, "multimem_all_gather": ar.multicast, "cases": {}}

    def timed(fn, iters):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) * 1e-3

    for T in (1, 16, 128, 1024, 4096):
        n = T * 8192
        x = torch.randn(n, generator=torch.Generator(device=dev).manual_seed(rank), device=dev).bfloat16()
        y = torch.empty_like(x)
        z = x.clone()
        iters = 200 if T <= 128 else 40
        t_fp8 = timed(lambda: ar.all_reduce(x, out=y), iters)
        t_nccl = timed(lambda: dist.all_reduce(z), iters)
        t_ws = timed(lambda: ar.all_reduce_in_workspace(x), iters)     # two-shot, result left in the workspace
        t_v2 = timed(lambda: ar.all_reduce(x, out=y, algo=3), iters)   # second variant: FP8 all-gather (one more quantisation)
        S, f = n * 2, 2 * (world - 1) / world
        out["cases"][f"T{T}"] = {"bytes": S, "fp8_us": round(t_fp8 * 1e6, 2), "nccl_bf16_us": round(t_nccl * 1e6, 2),
                                 "fp8_in_workspace_us": round(t_ws * 1e6, 2),
                                 "fp8_in_workspace_busbw": round(S / t_ws * f / 1e9, 1),
                                 "fp8_busbw": round(S / t_fp8 * f / 1e9, 1), "nccl_bf16_busbw": round(S / t_nccl * f / 1e9, 1),
                                 "ratio": round(t_nccl / t_fp8, 3),
                                 "fp8_gather_variant_us": round(t_v2 * 1e6, 2), "fp8_gather_variant_busbw": round(S / t_v2 * f / 1e9, 1),
                                 "fp8_gather_variant_ratio": round(t_nccl / t_v2, 3)}
    if R.lib().rdb_device_status() != 0:
        out["error"] = "device status word reports a timed-out wait"
    ar.close()
    return out


def run_single_other(args, torch, R, quant, dev):
    """Profiling aid for the other kernels: plain launches of one small case.
    dense_<n> (n^3; densesingle_<n> for the single-CTA kernel), sparse_M<m> (N=K=8192), reduce_<b>x<m>x<n>, quantize_T<t> ([t,8192] bf16, per-128 blocks), quantizept_T<t> (per tensor)."""
    one = torch.ones(1, device=dev)
    kind, _, arg = args.single.partition("_")
    reps = args.warmup + args.steps
    if kind in ("dense", "densesingle"):          # densesingle: the single-CTA 256 x 256 kernel instead of CTA pairs
        n = int(arg)
        tile_rows = 256 if kind == "densesingle" else 0
        A = torch.randint(0, 0x78, (n, n), dtype=torch.uint8, device=dev)
        B = torch.randint(0, 0x78, (n, n), dtype=torch.uint8, device=dev)
        D = torch.empty((n, n), dtype=torch.bfloat16, device=dev)
        for _ in range(reps):
            R.dense_gemm_fp8(A, B, one, one, out=D, tile_rows=tile_rows)
        work = {"flops_per_launch": 2.0 * n ** 3}
    elif kind == "sparse":
        M, N, K = int(arg[1:]), 8192, 8192
        packs = []
        for c in range(2):
            W = (torch.randn((N, K), generator=torch.Generator().manual_seed(c)) * 0.02).bfloat16()
            Wq, _ = quant.quantize_per_tensor(R.prune_2of4(W))
            v, m = R.pack_2of4(Wq)
            packs.append((v.to(dev), m.to(dev)))
        A = torch.randint(0, 0x78, (M, K), dtype=torch.uint8, device=dev)
        D = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
        for i in range(reps):
            R.sparse_gemm_fp8(A, packs[i % 2][0], packs[i % 2][1], one, one, out=D)
        work = {"algorithmic_bytes_per_launch": N * K // 2 + N * K // 8 + M * K + 2 * M * N}
    elif kind == "reduce":
        b, m, n = (int(x) for x in arg.split("x"))
        A = torch.rand((b, m, n), device=dev)
        B = torch.rand((b, m, n), device=dev)
        D = torch.empty((m, n), device=dev)
        for _ in range(reps):
            R.tiled_sum_reduce(A, B, D, b, m, n)
        work = {"algorithmic_bytes_per_launch": 8 * b * m * n + 4 * m * n}
    elif kind == "quantize":
        n = int(arg[1:]) * 8192
        x = torch.randn(n, device=dev).bfloat16()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        for i in range(reps):
            if i == args.warmup:
                ev[0].record()
            R.quantize_blocks128(x)
        ev[1].record()
        torch.cuda.synchronize()
        us = ev[0].elapsed_time(ev[1]) * 1e3 / max(1, args.steps)
        work = {"algorithmic_bytes_per_launch": n * 2 + n + n // 32, "us_per_launch": round(us, 2)}
    elif kind == "quantizept":
        n = int(arg[1:]) * 8192
        x = [torch.randn(n, device=dev).bfloat16() for _ in range(2)]
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        for i in range(reps):
            if i == args.warmup:
                ev[0].record()
            quant.quantize_per_tensor_device(x[i % 2])
        ev[1].record()
        torch.cuda.synchronize()
        us = ev[0].elapsed_time(ev[1]) * 1e3 / max(1, args.steps)
        # the tensor is read twice (maximum, then conversion); the second read may hit L2
        work = {"algorithmic_bytes_per_launch": n * 2 * 2 + n, "us_per_launch": round(us, 2),
                "gbs": round((n * 5) / us * 1e-3, 1)}
    else:
        raise SystemExit(f"unknown --single case {args.single}")
    torch.cuda.synchronize()
    print(json.dumps({"single": args.single, "launches": reps, **work}))


# ------------------------------------------------------- secondary suites
def _graph_time(torch, stream, fn, iters, reps=3):
    """Average device time (us) of fn(i) over a replayed CUDA graph of `iters` calls."""
    with torch.cuda.stream(stream):
        for i in range(2):
            fn(i)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            for i in range(iters):
                fn(i)
        g.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(reps):
            g.replay()
        b.record(stream)
        torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e3 / (reps * iters)


def run_suite(args):
    """Measured lines for the other paths of the scope table (one JSON line per
    invocation): dense GEMM (config 2, row-sharded over the ranks), 2:4 sparse
    GEMM (config 3), tiled_sum_reduce.  Not the headline metric."""
    import torch
    import torch.distributed as dist

    import rocm_dev_b200 as R
    from rocm_dev_b200 import quant

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=dev)
    stream = torch.cuda.Stream(device=dev)
    one = torch.ones(1, device=dev)
    peak_hbm, kind = measured_peak()
    out = {"suite": args.suite, "n_gpus": world, "data": "synthetic", "peak_kind": f"of {kind}"}

    def maxrank(us):
        if world == 1:
            return us
        t = torch.tensor([us], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    if args.suite == "dense":
        # config 2: M = N = K, the M rows of A and D split over the ranks, B replicated, no communication
        cases = {}
        for n in (4096, 8192, 16384):
            m_local = n // world
            g = torch.Generator(device=dev).manual_seed(n + rank)
            A = torch.randint(0, 0x78, (m_local, n), generator=g, dtype=torch.uint8, device=dev)
            B = torch.randint(0, 0x78, (n, n), generator=g, dtype=torch.uint8, device=dev)
            D = torch.empty((m_local, n), dtype=torch.bfloat16, device=dev)
            iters = 20 if n < 16384 else 4
            if world > 1:
                dist.barrier()
            us = maxrank(_graph_time(torch, stream, lambda i: R.dense_gemm_fp8(A, B, one, one, out=D), iters))
            lib_us = None
            try:
                a8, b8 = A.view(torch.float8_e4m3fn), B.view(torch.float8_e4m3fn).t()
                lib_us = maxrank(_graph_time(torch, stream, lambda i: torch._scaled_mm(a8, b8, scale_a=one, scale_b=one,
                                                                                      out_dtype=torch.bfloat16), iters))
            except Exception:  # noqa: BLE001
                pass
            tf = 2.0 * n * n * n / us / 1e6
            cases[str(n)] = {"us": round(us, 1), "tflops": round(tf, 1), "tflops_per_gpu": round(tf / world, 1),
                             "frac_of_4500_nominal_per_gpu": round(tf / world / 4500, 3),
                             "cublaslt_fp8_tflops": round(2.0 * n ** 3 / lib_us / 1e6, 1) if lib_us else None}
            del A, B, D
        out.update({"metric": "dense FP8 GEMM TFLOP/s (whole job)", "unit": "TFLOP/s", "scaling": "strong",
                    "config": {"workload": "configs[2]: M=N=K, rows of A/D sharded over ranks, no communication"},
                    "roofline": {"bound": "tensor", "peak": 4500.0, "unit": "TFLOP/s",
                                 "peak_kind": "nominal dense FP8; cuBLASLt FP8 on the same box listed per case"},
                    "cases": cases})
    elif args.suite == "sparse":
        N = K = 8192
        copies = 3
        g = torch.Generator().manual_seed(0)
        dense_w, packed = [], []
        for c in range(copies):
            W = (torch.randn((N, K), generator=g) * 0.02).bfloat16()
            Wq, _ = quant.quantize_per_tensor(R.prune_2of4(W))
            v, m = R.pack_2of4(Wq)
            dense_w.append(Wq.to(dev))
            packed.append((v.to(dev), m.to(dev)))
        cases = {}
        for M in (16, 64, 256):
            A = torch.randint(0, 0x78, (M, K), dtype=torch.uint8, device=dev)
            D = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
            sp = _graph_time(torch, stream, lambda i: R.sparse_gemm_fp8(A, packed[i % copies][0], packed[i % copies][1],
                                                                         one, one, out=D), 30)
            de = _graph_time(torch, stream, lambda i: R.dense_gemm_fp8(A, dense_w[i % copies], one, one, out=D), 30)
            sk = _graph_time(torch, stream, lambda i: R.skinny_gemm_fp8(A, dense_w[i % copies], one, one, out=D), 30) \
                if M <= 32 else None
            by = N * K // 2 + N * K // 8 + M * K + 2 * M * N
            best_dense = min(x for x in (de, sk) if x)
            cases[f"M{M}"] = {"sparse_us": round(sp, 2), "dense_gemm_us": round(de, 2),
                              "skinny_us": round(sk, 2) if sk else None, "speedup_vs_best_dense": round(best_dense / sp, 3),
                              "algorithmic_bytes": by, "gbs": round(by / sp / 1e3, 1),
                              "frac_of_hbm": round(by / sp / 1e3 / peak_hbm, 3),
                              "dense_equivalent_tflops": round(2.0 * M * N * K / sp / 1e6, 1)}
        out.update({"metric": "2:4 sparse FP8 GEMM time vs own dense kernels", "unit": "us",
                    "config": {"workload": "configs[3]: N=K=8192, M in {16,64,256}, 3 weight copies rotate (L2-cold)"},
                    "roofline": {"bound": "hbm", "peak": peak_hbm, "unit": "GB/s"}, "cases": cases})
    elif args.suite == "reduce":
        cases = {}
        for (b, m, n) in ((8, 4096, 4096), (32, 2048, 2048), (64, 512, 512)):
            A = torch.rand((b, m, n), device=dev)
            B = torch.rand((b, m, n), device=dev)
            D = torch.empty((m, n), device=dev)
            us = _graph_time(torch, stream, lambda i: R.tiled_sum_reduce(A, B, D, b, m, n), 10)
            by = 8 * b * m * n + 4 * m * n
            cases[f"{b}x{m}x{n}"] = {"us": round(us, 1), "gbs": round(by / us / 1e3, 1),
                                     "frac": round(by / us / 1e3 / peak_hbm, 3)}
        out.update({"metric": "tiled_sum_reduce HBM GB/s", "unit": "GB/s",
                    "roofline": {"bound": "hbm", "peak": peak_hbm, "unit": "GB/s"}, "cases": cases})
    elif args.suite == "allreduce":
        if world < 2:
            raise SystemExit("--suite allreduce needs torchrun with at least 2 ranks")
        out.update({"metric": "FP8-encoded allreduce busBW vs NCCL bf16", "unit": "GB/s",
                    "config": {"workload": "configs[4]: bf16 [T, 8192], T in {1,16,128,1024,4096}"},
                    "allreduce": bench_allreduce(torch, dist, R, dev, rank, world)})
    if R.lib().rdb_device_status() != 0:
        out["error"] = "device status word reports a timed-out wait"
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--single", default="", help="profiling aid: run one case, e.g. gate_up_M8, with plain launches")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-detail", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-allreduce", action="store_true")
    ap.add_argument("--suite", default="", choices=["", "dense", "sparse", "reduce", "allreduce"],
                    help="measure one of the other paths instead of the headline sweep")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.suite:
        run_suite(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
