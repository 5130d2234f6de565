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
# DRAM bytes (read + write) per algorithmic byte, each from one ncu capture of that kernel; DRAM traffic grows in
# proportion to the weight bytes, so the ratio is applied to the bytes of a launch.
TRAFFIC_PER_ALGO_BYTE = {"skinny_gemm_kernel": 1.03, "skinny_grouped_kernel": 1.028}
TRAFFIC_NOTE = {"skinny_gemm_kernel": "ncu capture of gate_up at M=8 (no split-K): 121.5 MB moved for 117.9 MB algorithmic; "
                                      "scaled by bytes",
                "skinny_grouped_kernel": "ncu capture of one grouped launch of the four projections at M=8: 225.0 MB moved for "
                                         "219.0 MB algorithmic; scaled by bytes"}
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
    few milliseconds on a thread while a region runs."""
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
                    time.sleep(0.002)
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
def make_inputs(torch, quant, dev, sets):
    """Synthetic operands with the value distribution of quantised N(0,1) /
    N(0,0.02) data.  weights[s][si]: `sets` independent copies of the four
    projection matrices (218 MB each set)."""
    weights = [[quant.synthetic_weights_fast(N, K, seed=100 * s + i, device=dev) for i, (_, N, K) in enumerate(SHAPES)]
               for s in range(sets)]
    acts = {}
    for M in MS:
        for K in sorted({k for _, _, k in SHAPES}):
            g = torch.Generator(device=dev).manual_seed(M * 131 + K)
            a = torch.randn((M, K), generator=g, device=dev)
            amax = a.abs().max()
            acts[(M, K)] = ((a * (448.0 / amax)).to(torch.float8_e4m3fn).view(torch.uint8), (amax / 448.0).reshape(1))
    outs = {(M, N): torch.empty((M, N), dtype=torch.bfloat16, device=dev) for M in MS for _, N, _ in SHAPES}
    return weights, acts, outs


def timed_graphs(torch, stream, graphs, steps, warmup, barrier=None, sampler=None):
    """Replays graphs[i % len] for `steps` timed iterations after `warmup`
    untimed ones; CUDA events on the launching stream.  Returns milliseconds."""
    with torch.cuda.stream(stream):
        if sampler:
            sampler.start()                  # clocks are sampled from the warm-up replays on: the same load, and
        for w in range(warmup):              # the timed region alone can be shorter than one sampling interval
            graphs[w % len(graphs)].replay()
        torch.cuda.synchronize()
        if barrier:
            barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.profiler.start()          # lets `ncu --profile-from-start off` see only the timed region
        e0.record(stream)
        for s in range(steps):
            graphs[s % len(graphs)].replay()
        e1.record(stream)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        if barrier:
            barrier()
        return e0.elapsed_time(e1)


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
    barrier = dist.barrier if world > 1 else None

    if args.single and not args.single.split("_M")[0] in [n for n, _, _ in SHAPES] + ["layer"]:
        return run_single_other(args, torch, R, quant, dev)

    # A grouped launch streams all of its problems at once, so each of them needs weights of its own for the
    # stream to stay L2-cold: one set of the four matrices per M, and two such groups alternating between steps.
    weights, acts, outs = make_inputs(torch, quant, dev, sets=2 if args.single else 2 * len(MS))
    flags = 0 if args.no_overlap else R.OVERLAP_PRIOR_KERNEL   # weights are never written inside the timed region

    def problems_of(M, wset):
        return [(acts[(M, K)][0], wset[si][0], acts[(M, K)][1], wset[si][1], outs[(M, N)])
                for si, (_, N, K) in enumerate(SHAPES)]

    if args.single:
        # profiling aid: plain launches of one case, weight copies rotating.  <shape>_M<m>: the per-call kernel;
        # layer_M<m>: the grouped kernel on the four projections of one layer
        name, m = args.single.rsplit("_M", 1)
        M = int(m)
        for i in range(args.warmup + args.steps):
            wset = weights[i % len(weights)]
            if name == "layer":
                assert R.skinny_gemm_fp8_grouped(problems_of(M, wset)) == 0
            else:
                si = [n for n, _, _ in SHAPES].index(name)
                Aq, sa = acts[(M, SHAPES[si][2])]
                R.skinny_gemm_fp8_tuned(Aq, wset[si][0], sa, wset[si][1], outs[(M, SHAPES[si][1])], 0, 0, 0, 0)
        torch.cuda.synchronize()
        by = sum(algo_bytes(M, N, K) for _, N, K in SHAPES) if name == "layer" else \
            algo_bytes(M, *SHAPES[[n for n, _, _ in SHAPES].index(name)][1:])
        print(json.dumps({"single": args.single, "launches": args.warmup + args.steps, "algorithmic_bytes_per_launch": by}))
        return

    # The sweep in three launch shapes (same GEMMs, same operands):
    #   grouped  one persistent launch for all 20 problems (rdb_skinny_gemm_fp8_grouped)        <- headline
    #   layer    one grouped launch per M: the four projections of a layer, 5 launches per step
    #   single   one rdb_skinny_gemm_fp8 launch per GEMM, 20 per step, programmatic dependent launch
    def step(mode, parity):
        half = len(MS)
        sets = weights[parity * half:(parity + 1) * half]
        if mode == "grouped":
            probs = [pr for mi, M in enumerate(MS) for pr in problems_of(M, sets[mi])]
            code = R.skinny_gemm_fp8_grouped(probs, flags)
            if code != 0:
                raise RuntimeError(f"grouped skinny GEMM returned {code}")
            return 1
        if mode == "layer":
            for mi, M in enumerate(MS):
                code = R.skinny_gemm_fp8_grouped(problems_of(M, sets[mi]), flags)
                if code != 0:
                    raise RuntimeError(f"grouped skinny GEMM returned {code}")
            return len(MS)
        n = 0
        for mi, M in enumerate(MS):
            for (Aq, Bq, sa, sb, D) in problems_of(M, sets[mi]):
                code = R.skinny_gemm_fp8_tuned(Aq, Bq, sa, sb, D, 0, 0, 0, flags)
                if code != 0:
                    raise RuntimeError(f"skinny GEMM returned {code}")
                n += 1
        return n

    stream = torch.cuda.Stream(device=dev)

    def graphs_of(mode):
        with torch.cuda.stream(stream):
            launches = step(mode, 0)
            torch.cuda.synchronize()
            gs = []
            for parity in range(2):          # two graphs (even / odd step) so that the weight groups alternate
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    step(mode, parity)
                gs.append(g)
        return gs, launches

    sampler = ClockSampler(local) if rank == 0 else None
    graphs, launches_per_step = graphs_of(args.mode)
    ms = timed_graphs(torch, stream, graphs, args.steps, max(args.warmup, 3), barrier, sampler)
    clocks = sampler.stop() if rank == 0 else None
    if R.lib().rdb_device_status() != 0:
        raise RuntimeError("device status word reports a timed-out wait")
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())

    # the other launch shapes, beside the headline (rank 0, fewer steps)
    modes = {args.mode: {"ms_per_step": round(ms / args.steps, 4), "launches_per_step": launches_per_step,
                         "gbs": round(step_bytes() * args.steps / ms / 1e6, 1)}}
    if rank == 0 and not args.no_detail:
        for mode in ("grouped", "layer", "single"):
            if mode in modes:
                continue
            gs, n = graphs_of(mode)
            k = max(4, min(args.steps, 50))
            t = timed_graphs(torch, stream, gs, k, 3)
            modes[mode] = {"ms_per_step": round(t / k, 4), "launches_per_step": n, "gbs": round(step_bytes() * k / t / 1e6, 1)}
            del gs

    # per-case detail (rank 0): each (shape, M) alone, L2-cold.  "grouped": lists of that one shape on distinct
    # weight copies (the reference's own timed region: BATCH launches of one shape on different B); "single":
    # one launch per GEMM, copies rotating
    detail = {}
    if rank == 0 and not args.no_detail:
        def act(M, K):
            if (M, K) not in acts:
                g = torch.Generator(device=dev).manual_seed(M * 131 + K)
                a = torch.randn((M, K), generator=g, device=dev)
                amax = a.abs().max()
                acts[(M, K)] = ((a * (448.0 / amax)).to(torch.float8_e4m3fn).view(torch.uint8), (amax / 448.0).reshape(1))
            return acts[(M, K)]
        for name, N, K, ms_list in [(n, N, K, MS) for n, N, K in SHAPES] + [("config0_8192x8192", 8192, 8192, [8])]:
            ncopies = min(32, max(8, -(-300_000_000 // (N * K))))     # >= 300 MB of distinct weights per list
            copies = [quant.synthetic_weights_fast(N, K, seed=977 + c, device=dev) for c in range(ncopies)]
            for M in ms_list:
                Aq, sa = act(M, K)
                D = outs.setdefault((M, N), torch.empty((M, N), dtype=torch.bfloat16, device=dev))
                one_list = [(Aq, c[0], sa, c[1], D) for c in copies]
                us_g = _graph_time(torch, stream, lambda i: R.skinny_gemm_fp8_grouped(one_list, flags), 2) / ncopies
                us_s = _graph_time(torch, stream, lambda i: R.skinny_gemm_fp8_tuned(Aq, copies[i % ncopies][0], sa, copies[0][1],
                                                                                    D, 0, 0, 0, flags), 24)
                by = algo_bytes(M, N, K)
                detail[f"{name}_M{M}"] = {"grouped_us": round(us_g, 2), "grouped_gbs": round(by / us_g / 1e3, 1),
                                          "single_us": round(us_s, 2), "single_gbs": round(by / us_s / 1e3, 1),
                                          "problems_per_grouped_launch": ncopies}
            del copies

    # end to end through the C ABI's host-buffer entry: every operand H2D, result D2H, each call
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
               "entry": "rdb_skinny_gemm_fp8_host (C ABI, host pointers)",
               "note": "weights, activations and scales copied from pinned host memory for every call"}
        # Beside it, the serving form of the same step: the weights are model state resident in HBM (set 0), the
        # step's inputs - every activation matrix and its scale - come from pinned host memory, all 20 GEMMs run as one
        # grouped launch, every result goes back to the host.  Reported as an extra key, not as the e2e value.
        dev_a = {k: (torch.empty_like(v[0], device=dev), torch.empty_like(v[1], device=dev)) for k, v in host_a.items()}

        def resident_step():
            for k, (ha, hs) in host_a.items():
                dev_a[k][0].copy_(ha, non_blocking=True)
                dev_a[k][1].copy_(hs, non_blocking=True)
            probs = [(dev_a[(M, K)][0], weights[0][si][0], dev_a[(M, K)][1], weights[0][si][1], outs[(M, N)])
                     for M in MS for si, (_, N, K) in enumerate(SHAPES)]
            if R.skinny_gemm_fp8_grouped(probs) != 0:
                raise RuntimeError("grouped skinny GEMM failed")
            for k, ho in host_o.items():
                ho.copy_(outs[k], non_blocking=True)
            torch.cuda.current_stream(dev).synchronize()
        resident_step()
        n_res = max(4, min(args.steps, 20))
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n_res):
            resident_step()
        b.record()
        torch.cuda.synchronize()
        res_ms = a.elapsed_time(b) / n_res
        e2e["weights_resident"] = {"value": step_bytes() / (res_ms * 1e-3) / 1e9, "unit": "GB/s (per GPU)", "ms_per_step": res_ms,
                                   "h2d_bytes_per_step": sum(M * K + 4 for M in MS for K in sorted({k for _, _, k in SHAPES})),
                                   "d2h_bytes_per_step": d2h, "steps": n_res,
                                   "note": "activations + scales H2D, one grouped launch on resident weights, results D2H; "
                                           "the same weights every step, so L2 may hold part of them"}

    sustained = None
    if rank == 0:
        # The timed region lasts a few milliseconds (one or two NVML samples, boost clocks).  The same replays, about
        # 150 ms of them, timed and sampled separately: what a long-running loop sees once the power cap has settled.
        # Run after the other skinny measurements of this line (they are taken in the state the headline was) and
        # before the weights the captured graphs read are released.
        extra = max(args.steps, min(2000, int(150.0 / max(ms / args.steps, 1e-3))))
        s2 = ClockSampler(local)
        with torch.cuda.stream(stream):
            s2.start()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for i in range(extra):
                graphs[i % len(graphs)].replay()
            e1.record(stream)
            torch.cuda.synchronize()
        sustained = {"steps": extra, "ms_per_step": e0.elapsed_time(e1) / extra, "clocks": s2.stop()}
    del weights
    torch.cuda.empty_cache()
    suites = None
    if not args.no_suites:
        suites = run_suites_compact(torch, dist, R, quant, dev, rank, world, stream)

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
    kernel = "skinny_gemm_kernel" if args.mode == "single" else "skinny_grouped_kernel"
    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp8_e4m3 x fp8_e4m3 -> f32", "data": "synthetic",
        "config": {"workload": "configs[1]: decode sweep M in {1,2,4,8,16} x {qkv,o,gate_up,down}",
                   "shapes": [[n, k] for _, n, k in SHAPES], "M": MS, "launches_per_step": launches_per_step,
                   "launch_shape": {"grouped": "all 20 GEMMs of the sweep in one persistent launch (rdb_skinny_gemm_fp8_grouped)",
                                    "layer": "one grouped launch per M (four projections), 5 per step",
                                    "single": "one launch per GEMM, 20 per step"}[args.mode],
                   "l2": "inputs larger than L2: every GEMM of a step has its own weight matrix (1.09 GB per step) and "
                         "two such groups alternate, so a matrix is re-read only after 2.2 GB of other weights",
                   "launch": "CUDA graph replay, programmatic dependent launch (weights are never written in the timed region)",
                   "multi_gpu": "replicas only"},
        "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s", "frac": per_gpu / peak,
                     "traffic": TRAFFIC_PER_ALGO_BYTE[kernel] * step_bytes() / launches_per_step,
                     "traffic_note": TRAFFIC_NOTE[kernel],
                     "peak_kind": f"of {peak_kind}", "kernel": kernel,
                     "algorithmic_bytes_per_launch": step_bytes() / launches_per_step,
                     "avg_launch_us": ms * 1e3 / (args.steps * launches_per_step)},
        "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches_per_step * args.steps, "clocks": clocks,
        "modes": modes, "detail": detail, "suites": suites,
    }
    if sustained is not None:           # rank 0's GPU alone; the same replays for ~150 ms
        gbs = step_bytes() / (sustained["ms_per_step"] * 1e-3) / 1e9
        line["sustained"] = {"steps": sustained["steps"], "ms_per_step": sustained["ms_per_step"], "gbs_per_gpu": gbs,
                             "frac": gbs / peak, "clocks": sustained["clocks"]}
    if allreduce is not None:
        line["allreduce"] = allreduce
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    if allreduce is not None and (not allreduce["parity"]["bit_exact"] or "error" in allreduce):
        raise SystemExit("allreduce: results differ from the oracle or a device wait timed out")


def allreduce_parity(torch, dist, R, ar, reg, dev, rank, world):
    """Outside every timed region: each variant of the allreduce on seeded
    per-rank inputs, this rank's result compared bit for bit with the CPU
    oracle (used here as the checker only).  Returns the parity block; the
    mismatch count is summed over the ranks."""
    import numpy as np
    from oracle import oracle as O
    O.build()
    from rocm_dev_b200.allreduce import ONE_SHOT, TWO_SHOT, TWO_SHOT_FP8_GATHER
    bits = lambda t: t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)  # noqa: E731
    cases, bad = 0, 0
    for T in (16, 1024):
        n = T * 8192
        xs = [torch.randn(n, generator=torch.Generator().manual_seed(9000 + 100 * T + r)).bfloat16() for r in range(world)]
        stacked = np.stack([bits(x) for x in xs])
        want = O.allreduce_fp8(stacked)[0]
        want_v2 = O.allreduce_fp8_regather(stacked)
        x = xs[rank].to(dev)
        runs = [("two_shot", lambda: ar.all_reduce(x, algo=TWO_SHOT), want),
                ("two_shot_in_workspace", lambda: ar.all_reduce_in_workspace(x), want),
                ("two_shot_registered", lambda: ar.all_reduce(x, out=reg[:n], algo=TWO_SHOT), want),
                ("automatic", lambda: ar.all_reduce(x), want),
                ("fp8_gather_variant", lambda: ar.all_reduce(x, algo=TWO_SHOT_FP8_GATHER), want_v2)]
        if n <= 1 << 20:
            runs.append(("one_shot", lambda: ar.all_reduce(x, algo=ONE_SHOT), want))
        for _name, fn, ref in runs:
            for _rep in range(2):                       # both staging sets
                got = bits(fn())
                bad += int((got != ref).sum())
                cases += 1
                dist.barrier()                          # a rank reads its result before any peer starts the next call
    t = torch.tensor([bad], dtype=torch.int64, device=dev)
    dist.all_reduce(t)
    total = int(t.item())
    return {"bit_exact": total == 0, "cases": cases, "mismatching_elements": total, "checker": "CPU oracle, T in {16, 1024}",
            "ranks": world}


def allreduce_graph_parity(torch, dist, arg, regg, dev, rank, world, so_far):
    """The oracle check for calls recorded in a CUDA graph: per size one graph of three calls (automatic into the
    registered buffer, two-shot into an ordinary buffer, second variant), replayed three times with new inputs."""
    import numpy as np
    from oracle import oracle as O
    bits = lambda t: t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)  # noqa: E731
    cases, bad = 0, 0
    for T in (16, 1024):
        n = T * 8192
        x = torch.zeros(n, dtype=torch.bfloat16, device=dev)
        y2, y3 = torch.empty_like(x), torch.empty_like(x)

        def issue():
            arg.all_reduce(x, out=regg[:n])
            arg.all_reduce(x, out=y2, algo=2)
            arg.all_reduce(x, out=y3, algo=3)
        issue()
        torch.cuda.synchronize()
        dist.barrier()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            issue()
        for rep in range(3):
            xs = [torch.randn(n, generator=torch.Generator().manual_seed(500 + 10 * rep + r + T)).bfloat16() for r in range(world)]
            x.copy_(xs[rank])
            g.replay()
            torch.cuda.synchronize()
            stacked = np.stack([bits(v) for v in xs])
            want = O.allreduce_fp8(stacked)[0]
            bad += int((bits(regg[:n]) != want).sum()) + int((bits(y2) != want).sum())
            bad += int((bits(y3) != O.allreduce_fp8_regather(stacked)).sum())
            cases += 3
            dist.barrier()
        del g
    t = torch.tensor([bad], dtype=torch.int64, device=dev)
    dist.all_reduce(t)
    total = int(t.item())
    return {"bit_exact": so_far["bit_exact"] and total == 0, "cases": so_far["cases"] + cases,
            "graph_replay_cases": cases, "mismatching_elements": so_far["mismatching_elements"] + total}


def bench_allreduce(torch, dist, R, dev, rank, world):
    """FP8-encoded allreduce against NCCL's bf16 allreduce on [T, 8192] bf16
    tensors.  busBW = S/t * 2(n-1)/n with S the bf16 size; device time, max over
    ranks.  Reported beside the headline metric when more than one GPU runs.
    Every variant is first checked bit for bit against the CPU oracle."""
    ar = R.Fp8AllReduce(max_elems=4096 * 8192, backend=os.environ.get("RDB_AR_BACKEND", "auto"))
    reg = ar.new_result_buffer(4096 * 8192)
    out = {"unit": "GB/s busBW", "world": world, "workspace": ar.backend, "multimem_all_gather": ar.multicast,
           "timing": "device time, max over ranks, median of 5 batches of back-to-back calls",
           "parity": allreduce_parity(torch, dist, R, ar, reg, dev, rank, world), "cases": {}}

    def timed(fn, iters, batches=5):
        """Median over `batches` batches of the per-call device time (each batch: events around `iters`
        back-to-back calls, max over ranks).  Single batches on these shared machines now and then come out
        twice as slow for whichever collective is running - NCCL's included - so one mean is not reported."""
        for _ in range(3):
            fn()
        per_batch = []
        for _ in range(batches):
            torch.cuda.synchronize()
            dist.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(iters):
                fn()
            b.record()
            torch.cuda.synchronize()
            per_batch.append(a.elapsed_time(b) / iters)
        t = torch.tensor(per_batch, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.median().item()) * 1e-3

    # the same calls recorded in a CUDA graph (a context that counts its calls on the device) and replayed: what a
    # graph-captured decode loop sees, without the per-call host path; NCCL's allreduce recorded the same way beside it
    arg = R.Fp8AllReduce(max_elems=4096 * 8192, backend="ipc", capturable=True)
    regg = arg.new_result_buffer(4096 * 8192)

    out["parity"].update(allreduce_graph_parity(torch, dist, arg, regg, dev, rank, world, out["parity"]))

    def timed_graph(fn, iters):
        try:
            fn()
            torch.cuda.synchronize()
            dist.barrier()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for _ in range(iters):
                    fn()
            t = timed(g.replay, 2) / iters
            del g
            return t
        except Exception as e:  # noqa: BLE001 - a collective library that cannot be captured here
            out.setdefault("graph_errors", []).append(f"{type(e).__name__}: {e}"[:160])
            return None

    for T in (1, 16, 128, 1024, 4096):
        n = T * 8192
        x = torch.randn(n, generator=torch.Generator(device=dev).manual_seed(rank), device=dev).bfloat16()
        y = torch.empty_like(x)
        z = x.clone()
        iters = 40 if T <= 128 else 10
        t_graph = timed_graph(lambda: arg.all_reduce(x, out=regg[:n]), iters)
        t_nccl_graph = timed_graph(lambda: dist.all_reduce(z), iters) if os.environ.get("RDB_BENCH_NCCL_GRAPH", "1") == "1" else None
        t_fp8 = timed(lambda: ar.all_reduce(x, out=y), iters)           # result into an ordinary buffer of the caller
        t_reg = timed(lambda: ar.all_reduce(x, out=reg[:n]), iters)     # result into the caller's registered buffer
        t_nccl = timed(lambda: dist.all_reduce(z), iters)
        t_ws = timed(lambda: ar.all_reduce_in_workspace(x), iters)     # two-shot, result left in the workspace
        t_v2 = timed(lambda: ar.all_reduce(x, out=y, algo=3), iters)   # second variant: FP8 all-gather (one more quantisation)
        S, f = n * 2, 2 * (world - 1) / world
        out["cases"][f"T{T}"] = {"bytes": S, "fp8_us": round(t_fp8 * 1e6, 2), "nccl_bf16_us": round(t_nccl * 1e6, 2),
                                 "fp8_registered_us": round(t_reg * 1e6, 2),
                                 "fp8_registered_busbw": round(S / t_reg * f / 1e9, 1),
                                 "registered_ratio": round(t_nccl / t_reg, 3),
                                 "fp8_in_workspace_us": round(t_ws * 1e6, 2),
                                 "fp8_in_workspace_busbw": round(S / t_ws * f / 1e9, 1),
                                 "fp8_busbw": round(S / t_fp8 * f / 1e9, 1), "nccl_bf16_busbw": round(S / t_nccl * f / 1e9, 1),
                                 "ratio": round(t_nccl / t_fp8, 3),
                                 "fp8_gather_variant_us": round(t_v2 * 1e6, 2), "fp8_gather_variant_busbw": round(S / t_v2 * f / 1e9, 1),
                                 "fp8_gather_variant_ratio": round(t_nccl / t_v2, 3),
                                 "fp8_graph_us": round(t_graph * 1e6, 2) if t_graph else None,
                                 "nccl_bf16_graph_us": round(t_nccl_graph * 1e6, 2) if t_nccl_graph else None,
                                 "graph_ratio": round(t_nccl_graph / t_graph, 3) if t_graph and t_nccl_graph else None}
    if R.lib().rdb_device_status() != 0:
        out["error"] = "device status word reports a timed-out wait"
    arg.close()
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


def _maxrank(torch, dist, dev, world, us):
    if world == 1:
        return us
    t = torch.tensor([us], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def suite_dense(torch, dist, R, dev, rank, world, stream, sizes=(4096, 8192, 16384)):
    """config 2: M = N = K, the M rows of A and D split over the ranks, B
    replicated, no communication; cuBLASLt FP8 (torch._scaled_mm) beside it as
    the library comparison."""
    one = torch.ones(1, device=dev)
    cases = {}
    for n in sizes:
        m_local = n // world
        g = torch.Generator(device=dev).manual_seed(n + rank)
        A = torch.randint(0, 0x78, (m_local, n), generator=g, dtype=torch.uint8, device=dev)
        B = torch.randint(0, 0x78, (n, n), generator=g, dtype=torch.uint8, device=dev)
        D = torch.empty((m_local, n), dtype=torch.bfloat16, device=dev)
        iters = 20 if n < 16384 else 4
        if world > 1:
            dist.barrier()
        us = _maxrank(torch, dist, dev, world, _graph_time(torch, stream, lambda i: R.dense_gemm_fp8(A, B, one, one, out=D), iters))
        lib_us = None
        try:
            a8, b8 = A.view(torch.float8_e4m3fn), B.view(torch.float8_e4m3fn).t()
            lib_us = _maxrank(torch, dist, dev, world,
                              _graph_time(torch, stream, lambda i: torch._scaled_mm(a8, b8, scale_a=one, scale_b=one,
                                                                                    out_dtype=torch.bfloat16), iters))
        except Exception:  # noqa: BLE001
            pass
        tf = 2.0 * n * n * n / us / 1e6
        cases[str(n)] = {"us": round(us, 1), "tflops": round(tf, 1), "tflops_per_gpu": round(tf / world, 1),
                         "frac_of_4500_nominal_per_gpu": round(tf / world / 4500, 3),
                         "cublaslt_fp8_tflops": round(2.0 * n ** 3 / lib_us / 1e6, 1) if lib_us else None}
        del A, B, D
    return {"metric": "dense FP8 GEMM TFLOP/s (whole job)", "unit": "TFLOP/s", "scaling": "strong",
            "config": {"workload": "configs[2]: M=N=K, rows of A/D sharded over ranks, no communication"},
            "roofline": {"bound": "tensor", "peak": 4500.0, "unit": "TFLOP/s",
                         "peak_kind": "nominal dense FP8; cuBLASLt FP8 on the same box listed per case"},
            "cases": cases}


def suite_sparse(torch, R, quant, dev, stream, ms=(16, 64, 256)):
    """config 3: N = K = 8192, weights pruned 2:4 and compressed; against the
    own dense kernels on the same pruned matrices."""
    one = torch.ones(1, device=dev)
    peak_hbm, _ = measured_peak()
    N = K = 8192
    copies = 6                      # 226 MB of compressed weights in rotation: nearly twice what L2 holds
    dense_w, packed = [], []
    for c in range(copies):
        g = torch.Generator(device=dev).manual_seed(c)
        W = (torch.randn((N, K), generator=g, device=dev) * 0.02).bfloat16()
        Wq, _ = quant.quantize_per_tensor(R.prune_2of4(W))          # pruning and quantising on the GPU (torch ops)
        v, m = R.pack_2of4(Wq.cpu())                                # the library's host packer
        dense_w.append(Wq)
        packed.append((v.to(dev), m.to(dev)))
        del W
    cases = {}
    for M in ms:
        A = torch.randint(0, 0x78, (M, K), dtype=torch.uint8, device=dev)
        D = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
        sp = _graph_time(torch, stream, lambda i: R.sparse_gemm_fp8(A, packed[i % copies][0], packed[i % copies][1],
                                                                     one, one, out=D), 30)
        # the same launches allowed to start while their predecessor drains (a decode loop: weights are constant)
        spo = _graph_time(torch, stream, lambda i: R.sparse_gemm_fp8(A, packed[i % copies][0], packed[i % copies][1],
                                                                      one, one, out=D, flags=R.OVERLAP_PRIOR_KERNEL), 30)
        de = _graph_time(torch, stream, lambda i: R.dense_gemm_fp8(A, dense_w[i % copies], one, one, out=D), 30)
        sk = _graph_time(torch, stream, lambda i: R.skinny_gemm_fp8(A, dense_w[i % copies], one, one, out=D), 30) \
            if M <= 32 else None
        by = N * K // 2 + N * K // 8 + M * K + 2 * M * N
        best_dense = min(x for x in (de, sk) if x)
        cases[f"M{M}"] = {"sparse_us": round(sp, 2), "dense_gemm_us": round(de, 2),
                          "skinny_us": round(sk, 2) if sk else None, "speedup_vs_best_dense": round(best_dense / sp, 3),
                          "algorithmic_bytes": by, "gbs": round(by / sp / 1e3, 1),
                          "frac_of_hbm": round(by / sp / 1e3 / peak_hbm, 3),
                          "sparse_overlapped_us": round(spo, 2), "overlapped_frac_of_hbm": round(by / spo / 1e3 / peak_hbm, 3),
                          "dense_equivalent_tflops": round(2.0 * M * N * K / sp / 1e6, 1)}
    # all copies as ONE launch (a list of GEMMs sharing the batch), per GEMM
    for M in ms[:2]:
        A = torch.randint(0, 0x78, (M, K), dtype=torch.uint8, device=dev)
        Ds = [torch.empty((M, N), dtype=torch.bfloat16, device=dev) for _ in range(copies)]
        probs = [(A, packed[c][0], packed[c][1], one, one, Ds[c]) for c in range(copies)]
        t = _graph_time(torch, stream, lambda i: R.sparse_gemm_fp8_grouped(probs), 10) / copies
        by = N * K // 2 + N * K // 8 + M * K + 2 * M * N
        cases[f"M{M}"].update({"list_us_per_gemm": round(t, 2), "list_frac_of_hbm": round(by / t / 1e3 / peak_hbm, 3)})
    return {"metric": "2:4 sparse FP8 GEMM time vs own dense kernels", "unit": "us",
            "config": {"workload": "configs[3]: N=K=8192, M in {16,64,256}, 6 weight copies rotate (L2-cold)"},
            "roofline": {"bound": "hbm", "peak": peak_hbm, "unit": "GB/s"}, "cases": cases}


def suite_reduce(torch, R, dev, stream, shapes=((8, 4096, 4096), (32, 2048, 2048), (64, 512, 512))):
    peak_hbm, _ = measured_peak()
    cases = {}
    for (b, m, n) in shapes:
        A = torch.rand((b, m, n), device=dev)
        B = torch.rand((b, m, n), device=dev)
        D = torch.empty((m, n), device=dev)
        us = _graph_time(torch, stream, lambda i: R.tiled_sum_reduce(A, B, D, b, m, n), 10)
        by = 8 * b * m * n + 4 * m * n
        cases[f"{b}x{m}x{n}"] = {"us": round(us, 1), "gbs": round(by / us / 1e3, 1), "frac": round(by / us / 1e3 / peak_hbm, 3)}
    return {"metric": "tiled_sum_reduce HBM GB/s", "unit": "GB/s",
            "roofline": {"bound": "hbm", "peak": peak_hbm, "unit": "GB/s"}, "cases": cases}


def suite_quant(torch, R, quant, dev, stream, T=16384):
    """The two quantisers on a [T, 8192] bf16 tensor (256 MB at T = 16384: larger than L2).
    Algorithmic bytes: read once + codes (+ scales) for the block encoder; the per-tensor
    quantiser must read the tensor twice (maximum first)."""
    peak_hbm, _ = measured_peak()
    n = T * 8192
    xs = [torch.randn(n, device=dev).bfloat16() for _ in range(2)]
    us_b = _graph_time(torch, stream, lambda i: R.quantize_blocks128(xs[i % 2]), 6)
    us_t = _graph_time(torch, stream, lambda i: quant.quantize_per_tensor_device(xs[i % 2]), 6)
    by_b, by_t = n * 2 + n + n // 32, n * 2 * 2 + n
    return {"metric": "bf16 -> e4m3 quantisers, HBM GB/s", "unit": "GB/s", "elements": n,
            "cases": {"blocks128": {"us": round(us_b, 1), "gbs": round(by_b / us_b / 1e3, 1), "frac": round(by_b / us_b / 1e3 / peak_hbm, 3)},
                      "per_tensor": {"us": round(us_t, 1), "gbs": round(by_t / us_t / 1e3, 1), "frac": round(by_t / us_t / 1e3 / peak_hbm, 3)}}}


def run_suites_compact(torch, dist, R, quant, dev, rank, world, stream):
    """The other kernels of the scope table in a few hundred milliseconds, for
    the headline line's `suites` key: dense 8192^3 (rows sharded over the ranks
    when there are several), and on rank 0 alone the 2:4 sparse GEMM, the
    sum-reduce and the two quantisers."""
    out = {"dense": suite_dense(torch, dist, R, dev, rank, world, stream, sizes=(4096, 8192))["cases"]}
    if rank == 0:
        out["sparse"] = suite_sparse(torch, R, quant, dev, stream)["cases"]
        out["tiled_sum_reduce"] = suite_reduce(torch, R, dev, stream, shapes=((8, 4096, 4096),))["cases"]
        out["quantize"] = suite_quant(torch, R, quant, dev, stream)["cases"]
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    return out


def run_suite(args):
    """Measured lines for the other paths of the scope table (one JSON line per
    invocation): dense GEMM (config 2, row-sharded over the ranks), 2:4 sparse
    GEMM (config 3), tiled_sum_reduce, the quantisers, the allreduce.  Not the
    headline metric."""
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
    _, kind = measured_peak()
    out = {"suite": args.suite, "n_gpus": world, "data": "synthetic", "peak_kind": f"of {kind}"}
    if args.suite == "dense":
        out.update(suite_dense(torch, dist, R, dev, rank, world, stream))
    elif args.suite == "sparse":
        out.update(suite_sparse(torch, R, quant, dev, stream))
    elif args.suite == "reduce":
        out.update(suite_reduce(torch, R, dev, stream))
    elif args.suite == "quant":
        out.update(suite_quant(torch, R, quant, dev, stream))
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
    if "allreduce" in out and (not out["allreduce"]["parity"]["bit_exact"] or "error" in out["allreduce"]):
        raise SystemExit("allreduce: results differ from the oracle or a device wait timed out")


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
    ap.add_argument("--no-overlap", action="store_true", help="plain launches instead of programmatic dependent launch")
    ap.add_argument("--no-suites", action="store_true", help="skip the compact dense / sparse / reduce / quantiser block")
    ap.add_argument("--mode", default="grouped", choices=["grouped", "layer", "single"],
                    help="launch shape of the headline sweep (the other two are reported beside it in `modes`)")
    ap.add_argument("--suite", default="", choices=["", "dense", "sparse", "reduce", "quant", "allreduce"],
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
