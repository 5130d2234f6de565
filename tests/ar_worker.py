"""One rank of the multi-GPU allreduce test (launched by test_allreduce.py):
runs the FP8-encoded allreduce for several sizes and both algorithms and
compares every result, bit for bit, with the CPU oracle."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    backend = os.environ.get("RDB_AR_BACKEND", "ipc")
    if backend == "ipc":
        dist.init_process_group("gloo")      # handles travel over gloo; the data path is the library's own
    else:
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    import rocm_dev_b200 as R
    from oracle import oracle as O
    try:
        ar = R.Fp8AllReduce(max_elems=4096 * 8192, backend=backend)
    except Exception as e:  # noqa: BLE001  - no symmetric memory in this build of torch: the IPC workspace is the fallback
        if backend != "symm":
            raise
        print(f"rank {rank}: symmetric memory unavailable ({type(e).__name__}), using ipc")
        ar = R.Fp8AllReduce(max_elems=4096 * 8192, backend="ipc")
    print(f"rank {rank} backend {ar.backend} multicast {ar.multicast}")
    dev = torch.device("cuda", rank)
    cases = [(128, 1), (8192, 1), (8192, 2), (16 * 8192, 0), (128 * 8192, 2), (640, 2), (1024 * 8192, 0), (4096 * 8192, 2),
             (513 * 8192 + 128, 2), (640, 3), (128 * 8192, 3), (513 * 8192 + 128, 3)]
    for n, algo in cases:
        for rep in range(2):                 # twice: both staging sets, growing epochs
            xs = [torch.randn(n, generator=torch.Generator().manual_seed(1000 * rep + 17 * r + n)).bfloat16()
                  for r in range(world)]
            out = ar.all_reduce(xs[rank].to(dev), algo=algo)
            torch.cuda.synchronize()
            assert R.lib().rdb_device_status() == 0, "device-side wait timed out"
            bits = np.stack([x.view(torch.int16).numpy().view(np.uint16) for x in xs])
            want = O.allreduce_fp8_regather(bits) if algo == 3 else O.allreduce_fp8(bits)[0]
            got = out.cpu().view(torch.int16).numpy().view(np.uint16)
            assert np.array_equal(got, want), f"rank {rank} n {n} algo {algo} rep {rep}: {(got != want).sum()} differ"
            if algo == 2:                    # the same result left in the workspace (no copy-out)
                view = ar.all_reduce_in_workspace(xs[rank].to(dev))
                torch.cuda.synchronize()
                assert np.array_equal(view.cpu().view(torch.int16).numpy().view(np.uint16), want)
    # results delivered straight into registered buffers (no copy out of the workspace)
    reg = ar.new_result_buffer(4096 * 8192)
    for n, off in ((8192, 0), (128 * 8192, 1 << 20), (513 * 8192 + 128, 0), (4096 * 8192, 0)):
        for rep in range(2):
            xs = [torch.randn(n, generator=torch.Generator().manual_seed(7000 * rep + 13 * r + n)).bfloat16()
                  for r in range(world)]
            out = ar.all_reduce(xs[rank].to(dev), out=reg[off:off + n], algo=2)
            torch.cuda.synchronize()
            assert R.lib().rdb_device_status() == 0, "device-side wait timed out"
            want = O.allreduce_fp8(np.stack([x.view(torch.int16).numpy().view(np.uint16) for x in xs]))[0]
            got = out.cpu().view(torch.int16).numpy().view(np.uint16)
            assert np.array_equal(got, want), f"rank {rank} registered n {n} rep {rep}: {(got != want).sum()} differ"
            dist.barrier()               # nobody starts the next call while a rank still reads this result
    # row-parallel linear + allreduce with the GEMM epilogue feeding the staging area: K split over the ranks
    from rocm_dev_b200 import quant
    for (M, N, K) in ((8, 4096, 4096), (16, 1024, 2048 * world), (32, 6144, 1024 * world)):
        Aq, Bq, sa, sb = quant.synthetic_gemm_operands(M, N, K, seed=world + M)
        kr = K // world
        sl = [(Aq[:, r * kr:(r + 1) * kr].contiguous().to(dev), Bq[:, r * kr:(r + 1) * kr].contiguous().to(dev)) for r in range(world)]
        dsa, dsb = sa.to(dev), sb.to(dev)
        partial = []
        for r in range(world):                           # every rank's partial product, computed here with the same kernel
            D = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
            assert R.skinny_gemm_fp8_grouped([(sl[r][0], sl[r][1], dsa, dsb, D)]) == 0
            partial.append(D.reshape(-1).cpu().view(torch.int16).numpy().view(np.uint16))
        want = O.allreduce_fp8(np.stack(partial))[0]
        for rep in range(2):
            out = ar.skinny_gemm_all_reduce(sl[rank][0], sl[rank][1], dsa, dsb)
            torch.cuda.synchronize()
            assert R.lib().rdb_device_status() == 0, "device-side wait timed out"
            got = out.reshape(-1).cpu().view(torch.int16).numpy().view(np.uint16)
            assert np.array_equal(got, want), f"rank {rank} fused linear {M}x{N}x{K} rep {rep}: {(got != want).sum()} differ"
            dist.barrier()
    dist.barrier()
    ar.close()
    # calls counted on the device, recorded in a CUDA graph and replayed with new inputs (three calls per replay, so the
    # staging sets alternate between replays), then a direct call on the same object
    cap = R.Fp8AllReduce(max_elems=1024 * 8192, backend="ipc", capturable=True)
    sizes = (16 * 8192, 1024 * 8192, 513 * 1024 + 128)
    xd = [torch.zeros(n, dtype=torch.bfloat16, device=dev) for n in sizes]
    od = [torch.empty(n, dtype=torch.bfloat16, device=dev) for n in sizes]
    algos = (1, 2, 3)

    def inputs(rep):
        return [[torch.randn(n, generator=torch.Generator().manual_seed(31 * rep + 7 * r + n)).bfloat16() * (rep + 1)
                 for r in range(world)] for n in sizes]

    def check_outputs(xs, what):
        torch.cuda.synchronize()
        assert R.lib().rdb_device_status() == 0, "device-side wait timed out"
        for i, algo in enumerate(algos):
            bits = np.stack([x.view(torch.int16).numpy().view(np.uint16) for x in xs[i]])
            want = O.allreduce_fp8_regather(bits) if algo == 3 else O.allreduce_fp8(bits)[0]
            got = od[i].cpu().view(torch.int16).numpy().view(np.uint16)
            assert np.array_equal(got, want), f"rank {rank} {what} size {sizes[i]} algo {algo}: {(got != want).sum()} differ"
        dist.barrier()

    xs = inputs(0)
    for i, algo in enumerate(algos):
        xd[i].copy_(xs[i][rank])
        cap.all_reduce(xd[i], out=od[i], algo=algo)          # before the capture: per-device set-up
    check_outputs(xs, "direct")
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for i, algo in enumerate(algos):
                cap.all_reduce(xd[i], out=od[i], algo=algo)
    torch.cuda.current_stream().wait_stream(side)
    for rep in range(1, 5):
        xs = inputs(rep)
        for i in range(len(sizes)):
            xd[i].copy_(xs[i][rank])
            od[i].zero_()
        graph.replay()
        check_outputs(xs, f"replay {rep}")
    xs = inputs(9)
    for i, algo in enumerate(algos):
        xd[i].copy_(xs[i][rank])
        cap.all_reduce(xd[i], out=od[i], algo=algo)
    check_outputs(xs, "direct after replays")
    del graph
    cap.close()
    dist.destroy_process_group()
    print(f"rank {rank} ok")


if __name__ == "__main__":
    main()
