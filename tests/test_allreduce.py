"""FP8-encoded allreduce.  The encoding must be bit-exact; because the kernels
round the product and the rank-ordered sum separately, as the oracle does, the
reduced bf16 result is compared bit for bit as well (stricter than the stated
tolerance of 1e-2 relative Frobenius / 2 bf16 ulp)."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bits(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


# ------------------------------------------------------------- CPU (gloo)
def _gloo_rank(rank, world, port, n, q):
    """The protocol of the two-shot algorithm acted out by CPU ranks with the
    oracle's arithmetic: encode, scatter shards, reduce in rank order, gather."""
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    from oracle import oracle as O
    from rocm_dev_b200.allreduce import GROUP, shard_groups
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    x = torch.randn(n, generator=torch.Generator().manual_seed(rank)).bfloat16()
    enc_q, enc_s = O.quantize_blocks128(_bits(x))
    qs = [torch.empty(n, dtype=torch.uint8) for _ in range(world)]
    ss = [torch.empty(n // 128) for _ in range(world)]
    dist.all_gather(qs, torch.from_numpy(enc_q))
    dist.all_gather(ss, torch.from_numpy(enc_s))
    gb, ge = shard_groups(n, world)[rank]
    lo, hi = gb * GROUP, min(ge * GROUP, n)
    acc = np.zeros(hi - lo, np.float32)
    for r in range(world):                    # rank order; product and sum rounded separately
        deq = (O.e4m3fn_decode(qs[r].numpy()[lo:hi]) * np.repeat(ss[r].numpy()[lo // 128:hi // 128], 128)).astype(np.float32)
        acc = (acc + deq).astype(np.float32)
    mine = torch.from_numpy(O.bf16_encode(acc).astype(np.int32))
    sizes = [min(e * GROUP, n) - b * GROUP for b, e in shard_groups(n, world)]
    parts = [torch.empty(s, dtype=torch.int32) for s in sizes]
    dist.all_gather(parts, mine) if len(set(sizes)) == 1 else dist.all_gather_object(parts, mine)
    q.put((rank, torch.cat([p if isinstance(p, torch.Tensor) else p for p in parts]).numpy().astype(np.uint16)))
    dist.destroy_process_group()


@pytest.mark.parametrize("n", [1024, 128 * 37])
def test_two_rank_protocol_on_cpu(oracle, n):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() + n) % 1000
    procs = [ctx.Process(target=_gloo_rank, args=(r, 2, port, n, q)) for r in range(2)]
    [p.start() for p in procs]
    res = dict(q.get(timeout=120) for _ in range(2))
    [p.join(timeout=60) for p in procs]
    xs = np.stack([_bits(torch.randn(n, generator=torch.Generator().manual_seed(r)).bfloat16()) for r in range(2)])
    want, _, _ = oracle.allreduce_fp8(xs)
    assert np.array_equal(res[0], want) and np.array_equal(res[1], want)


def _gloo_rank_that_may_leave(rank, world, port, q):
    """Rank 1 leaves before the handle exchange; rank 0 must get an error from the process group instead of waiting
    for ever (the host-side form of a failed peer: nothing on a GPU is involved)."""
    import datetime
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    if rank == 1:
        q.put((1, "left"))
        q.close()
        q.join_thread()                          # the message is out; now disappear without a clean shutdown
        os._exit(0)
    try:
        handles = [None] * world
        dist.all_gather_object(handles, b"x" * 64)          # the exchange Fp8AllReduce's set-up performs
        q.put((0, "no error"))
    except Exception as e:  # noqa: BLE001
        q.put((0, "error: " + type(e).__name__))


def test_a_rank_that_leaves_before_set_up_is_an_error_not_a_hang():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + os.getpid() % 200
    procs = [ctx.Process(target=_gloo_rank_that_may_leave, args=(r, 2, port, q)) for r in range(2)]
    [p.start() for p in procs]
    res = dict(q.get(timeout=60) for _ in range(2))
    [p.join(timeout=30) for p in procs]
    assert res[1] == "left" and res[0].startswith("error"), res


def test_shard_groups_cover_every_group_once():
    from rocm_dev_b200.allreduce import shard_groups
    for n in (128, 512, 640, 8192, 8192 * 4096, 128 * 999):
        for w in range(1, 9):
            sh = shard_groups(n, w)
            assert sh[0][0] == 0 and sh[-1][1] == (n + 511) // 512
            assert all(a[1] == b[0] for a, b in zip(sh, sh[1:]))
            assert max(e - b for b, e in sh) - min(e - b for b, e in sh) <= 1


# ------------------------------------------------------------------ GPU
@pytest.mark.gpu
@pytest.mark.parametrize("n", [128, 512, 640, 8192, 128 * 1001])
def test_encoder_is_bit_exact(cuda_device, oracle, n):
    import rocm_dev_b200 as R
    x = torch.randn(n, generator=torch.Generator().manual_seed(n)).bfloat16()
    x[:128] = 0                                            # an all-zero block: scale 1
    if n > 300:
        x[200] = 3.0e38
        x[300] = -1.0e-30
    q, s = R.quantize_blocks128(x.to(cuda_device))
    wq, ws = oracle.quantize_blocks128(_bits(x))
    assert np.array_equal(q.cpu().numpy(), wq)
    assert np.array_equal(s.cpu().numpy().view(np.uint32), ws.view(np.uint32))


@pytest.mark.gpu
def test_encoder_bit_exact_on_many_blocks_and_magnitudes(cuda_device, oracle):
    """A million blocks whose magnitudes span 2^-120 .. 2^120: scales and codes
    equal the oracle's (which divides with IEEE divisions)."""
    import rocm_dev_b200 as R
    nb = 1 << 14
    g = torch.Generator().manual_seed(42)
    mag = torch.exp2(torch.randint(-120, 121, (nb, 1), generator=g).float())
    x = (torch.randn(nb, 128, generator=g) * mag).bfloat16().reshape(-1)
    q, s = R.quantize_blocks128(x.to(cuda_device))
    wq, ws = oracle.quantize_blocks128(_bits(x))
    assert np.array_equal(s.cpu().numpy().view(np.uint32), ws.view(np.uint32))
    assert np.array_equal(q.cpu().numpy(), wq)


@pytest.mark.gpu
def test_encoder_division_is_the_ieee_quotient(cuda_device):
    """The encoder divides by multiplying with a rounded reciprocal and one
    residual correction; for every bf16 x and a wide set of divisors (random,
    powers of two, all-ones and near-all-ones significands, tiny, huge, inf,
    the amax/448 values of real blocks) the e4m3 encoding - and every normal fp32 quotient - equals that of x / s,
    over all x a block with that scale can contain."""
    import rocm_dev_b200 as R
    g = torch.Generator().manual_seed(0)
    rnd = (torch.randn(20000, generator=g).abs() + 1e-3) * torch.exp2(torch.randint(-40, 40, (20000,), generator=g).float())
    real = torch.randn(4096, 128, generator=g).bfloat16().float().abs().amax(1) / 448.0
    special_bits = [0x3F800000, 0x3FFFFFFF, 0x3FFFFFFE, 0x3F800001, 0x00800000, 0x7F7FFFFF, 0x7F800000, 0x0D000000,
                    0x0E000001, 0x71000000, 0x717FFFFF, 0x3B124925, 0x3C000000, 0x3EAAAAAB, 0x40490FDB]
    special = torch.tensor(special_bits, dtype=torch.int32).view(torch.float32)
    ones = (torch.arange(60, 200, dtype=torch.int32) << 23 | 0x7FFFFF).view(torch.float32)
    s = torch.cat([rnd, real, special, ones, ones.view(torch.int32).sub(1).view(torch.float32)]).to(cuda_device)
    bad = torch.zeros(2, dtype=torch.int64, device=cuda_device)
    assert R.lib().rdb_debug_division_mismatches(s.data_ptr(), s.numel(), bad.data_ptr(), 0) == 0
    torch.cuda.synchronize()
    assert bad[0].item() == 0, f"{bad[0].item()} encodings differ from those of the IEEE quotient"
    assert bad[1].item() == 0, f"{bad[1].item()} normal fp32 quotients differ from IEEE division"


@pytest.mark.gpu
@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("algo", [1, 2])
def test_emulated_ranks_on_one_gpu(cuda_device, oracle, world, algo):
    import rocm_dev_b200 as R
    lr = R.LocalRanks(world, max_elems=1 << 20, device=cuda_device)
    try:
        for n in (128, 640, 8192, 128 * 517, 1 << 20):
            for rep in range(2):
                xs = [torch.randn(n, generator=torch.Generator().manual_seed(100 * rep + r)).bfloat16() for r in range(world)]
                outs = lr.all_reduce([x.to(cuda_device) for x in xs], algo=algo)
                torch.cuda.synchronize()
                assert R.lib().rdb_device_status() == 0
                want, _, _ = oracle.allreduce_fp8(np.stack([_bits(x) for x in xs]))
                for r in range(world):
                    assert np.array_equal(_bits(outs[r]), want), (world, algo, n, rep, r)
    finally:
        lr.close()


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4, 8])
def test_automatic_choice_at_the_one_shot_limit(cuda_device, oracle, world):
    """The largest message the automatic choice still sends one-shot (2^22 elements on up to four ranks, 2^21 on
    more), one block less, and one block more (two-shot): all bit-exact."""
    import rocm_dev_b200 as R
    limit = (1 << 22) if world <= 4 else (1 << 21)
    lr = R.LocalRanks(world, max_elems=limit + 128, device=cuda_device)
    try:
        for n in (limit - 128, limit, limit + 128):
            xs = [torch.randn(n, generator=torch.Generator().manual_seed(3 * r + n % 1000)).bfloat16() for r in range(world)]
            outs = lr.all_reduce([x.to(cuda_device) for x in xs], algo=0)
            torch.cuda.synchronize()
            assert R.lib().rdb_device_status() == 0
            want, _, _ = oracle.allreduce_fp8(np.stack([_bits(x) for x in xs]))
            for r in range(world):
                assert np.array_equal(_bits(outs[r]), want), (world, n, r)
    finally:
        lr.close()


@pytest.mark.gpu
def test_a_second_context_over_a_used_workspace(cuda_device, oracle):
    """Epochs restart with a new context: what earlier calls left in the workspace (flag words, lines whose valid
    mark is an epoch) must not pass for the new context's calls of the same number."""
    import rocm_dev_b200 as R
    from rocm_dev_b200.allreduce import _create
    world, n = 2, 128 * 33
    lr = R.LocalRanks(world, max_elems=1 << 16, device=cuda_device)
    try:
        def run(seed, algo):
            xs = [torch.randn(n, generator=torch.Generator().manual_seed(seed + r)).bfloat16() for r in range(world)]
            outs = lr.all_reduce([x.to(cuda_device) for x in xs], algo=algo)
            torch.cuda.synchronize()
            want, _, _ = oracle.allreduce_fp8(np.stack([_bits(x) for x in xs]))
            return all(np.array_equal(_bits(o), want) for o in outs)
        for algo in (1, 2, 1, 2):
            assert run(10 * algo, algo)
        torch.cuda.synchronize()
        for c in lr.ctx:
            R.lib().rdb_ar_destroy(c)
        with torch.cuda.device(cuda_device):
            ptrs = [w.ptr for w in lr.ws]
            lr.ctx = [_create(r, world, ptrs, 1 << 16) for r in range(world)]       # epochs are back at zero
        for algo in (1, 2, 1, 2):
            assert run(100 + 7 * algo, algo)                                          # different data, same call numbers
        assert R.lib().rdb_device_status() == 0
    finally:
        lr.close()


def test_regather_variant_oracle_properties(oracle):
    """The FP8-all-gather variant is decode(encode(first variant)): idempotent
    (a second round trip changes nothing), exact on zero blocks, and within one
    e4m3 rounding step (2^-4 relative to the block maximum's binade) of the first variant."""
    n = 128 * 9
    xs = np.stack([_bits(torch.randn(n, generator=torch.Generator().manual_seed(r)).bfloat16()) for r in range(4)])
    xs[:, :128] = 0
    v1, _, _ = oracle.allreduce_fp8(xs)
    v2 = oracle.allreduce_fp8_regather(xs)
    assert not v2[:128].any()
    q, s = oracle.quantize_blocks128(v2)
    again = oracle.bf16_encode(oracle.e4m3fn_decode(q).astype(np.float32) * np.repeat(s, 128))
    assert np.array_equal(again, v2)
    a, b = oracle.bf16_decode(v1).reshape(-1, 128), oracle.bf16_decode(v2).reshape(-1, 128)
    amax = np.abs(a).max(axis=1, keepdims=True)
    assert (np.abs(a - b) <= amax / 16 + 1e-30).all()


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 3, 8])
def test_emulated_ranks_fp8_all_gather_variant(cuda_device, oracle, world):
    """algo 3: the reduced shard is block-quantised again for the all-gather;
    bit-exact against the oracle's composition of the same primitives."""
    import rocm_dev_b200 as R
    from rocm_dev_b200.allreduce import TWO_SHOT_FP8_GATHER
    lr = R.LocalRanks(world, max_elems=1 << 20, device=cuda_device)
    try:
        for n in (128, 640, 128 * 517, 1 << 20):
            for rep in range(2):
                xs = [torch.randn(n, generator=torch.Generator().manual_seed(7 * rep + r)).bfloat16() * (1 + 10 * r) for r in range(world)]
                outs = lr.all_reduce([x.to(cuda_device) for x in xs], algo=TWO_SHOT_FP8_GATHER)
                torch.cuda.synchronize()
                assert R.lib().rdb_device_status() == 0
                want = oracle.allreduce_fp8_regather(np.stack([_bits(x) for x in xs]))
                for r in range(world):
                    assert np.array_equal(_bits(outs[r]), want), (world, n, rep, r)
                # a first-variant call in between must still be exact (the two share the gather area)
                outs = lr.all_reduce([x.to(cuda_device) for x in xs], algo=2)
                want1, _, _ = oracle.allreduce_fp8(np.stack([_bits(x) for x in xs]))
                assert np.array_equal(_bits(outs[0]), want1)
    finally:
        lr.close()


@pytest.mark.gpu
def test_full_size_properties(cuda_device, oracle):
    """64 MB per rank (T = 4096 rows of 8192): close to the exact sum, identical
    on all ranks, and scaling the inputs by a power of two scales the result."""
    import rocm_dev_b200 as R
    world, n = 4, 4096 * 8192
    lr = R.LocalRanks(world, max_elems=n, device=cuda_device)
    try:
        xs = [torch.randn(n, generator=torch.Generator(device=cuda_device).manual_seed(r), device=cuda_device).bfloat16()
              for r in range(world)]
        outs = lr.all_reduce(xs, algo=2)
        exact = sum(x.float() for x in xs)
        rel = (outs[0].float() - exact).norm() / exact.norm()
        assert rel < 5e-2                                   # two e4m3 roundings per term, not an exact sum
        assert all(torch.equal(outs[0], o) for o in outs[1:])
        outs4 = lr.all_reduce([4 * x for x in xs], algo=2)
        assert torch.equal(outs4[0].float(), 4 * outs[0].float())
        rows = slice(0, 8192 * 3)                           # the oracle on the first rows
        want, _, _ = oracle.allreduce_fp8(np.stack([_bits(x[rows]) for x in xs]))
        assert np.array_equal(_bits(outs[0][rows]), want)
    finally:
        lr.close()


@pytest.mark.gpu
def test_fused_call_on_one_rank_and_its_trace(cuda_device, oracle):
    """World size 1 through the fused single-launch entry (the multi-rank form of
    the same kernel runs in the multi-GPU tests), with the step trace switched on:
    stamps are ordered and the result equals the oracle's."""
    import rocm_dev_b200 as R
    from rocm_dev_b200.allreduce import _Workspace, _create
    from rocm_dev_b200._lib import check
    n = 128 * 4099
    with torch.cuda.device(cuda_device):
        ws = _Workspace(1, n)
        ctx = _create(0, 1, [ws.ptr], n)
        trace = torch.zeros(16, dtype=torch.int64, device=cuda_device)
        check(R.lib().rdb_ar_set_trace(ctx, trace.data_ptr()), "rdb_ar_set_trace")
        x = torch.randn(n, generator=torch.Generator().manual_seed(5)).bfloat16()
        xd, out = x.to(cuda_device), torch.empty(n, dtype=torch.bfloat16, device=cuda_device)
        stream = torch.cuda.current_stream().cuda_stream
        for algo, want in ((2, oracle.allreduce_fp8(_bits(x)[None])[0]), (3, oracle.allreduce_fp8_regather(_bits(x)[None]))):
            check(R.lib().rdb_ar_allreduce(ctx, xd.data_ptr(), out.data_ptr(), n, algo, stream), "rdb_ar_allreduce")
            torch.cuda.synchronize()
            assert R.lib().rdb_device_status() == 0
            assert np.array_equal(_bits(out), want)
            t = trace.cpu().numpy()
            assert (np.diff(t[:6]) >= 0).all() and t[0] > 0 and (np.diff(t[8:14]) >= 0).all()
        check(R.lib().rdb_ar_set_trace(ctx, None), "rdb_ar_set_trace")
        R.lib().rdb_ar_destroy(ctx)
        ws.free()


@pytest.mark.gpu
def test_calls_recorded_in_a_cuda_graph(cuda_device, oracle):
    """A context that counts its calls on the device: three allreduce calls (one-shot, two-shot, second variant) and a
    GEMM + allreduce are recorded once and replayed with new inputs in the recorded buffers; every replay - an odd
    number of calls each, so the staging sets alternate between replays - equals the oracle bit for bit, direct calls
    in between included.  World size 1 here; the multi-rank form runs in the multi-GPU tests."""
    import rocm_dev_b200 as R
    from rocm_dev_b200 import quant
    from rocm_dev_b200.allreduce import _Workspace, _create
    from rocm_dev_b200.skinny_gemm import _problem_array
    from rocm_dev_b200._lib import check
    L = R.lib()
    n, (M, N, K) = 128 * 1031, (8, 1024, 2048)
    with torch.cuda.device(cuda_device):
        ws = _Workspace(1, n)
        ctx = _create(0, 1, [ws.ptr], n)
        check(L.rdb_ar_set_device_epoch(ctx, 1), "rdb_ar_set_device_epoch")
        assert L.rdb_ar_begin_call(ctx) == -1                                   # the separate phases need the host's count
        xd = torch.zeros(n, dtype=torch.bfloat16, device=cuda_device)
        outs = [torch.empty(n, dtype=torch.bfloat16, device=cuda_device) for _ in range(3)]
        Aq, Bq, sa, sb = quant.synthetic_gemm_operands(M, N, K, seed=3)
        A, B, dsa, dsb = Aq.to(cuda_device), Bq.to(cuda_device), sa.to(cuda_device), sb.to(cuda_device)
        D = torch.empty((M, N), dtype=torch.bfloat16, device=cuda_device)
        lin = torch.empty((M, N), dtype=torch.bfloat16, device=cuda_device)
        assert R.skinny_gemm_fp8_grouped([(A, B, dsa, dsb, D)]) == 0
        torch.cuda.synchronize()
        want_lin = oracle.allreduce_fp8(_bits(D.reshape(-1))[None])[0]
        arr = _problem_array([(A, B, dsa, dsb, lin)])

        def issue(stream):
            for algo, o in zip((1, 2, 3), outs):
                check(L.rdb_ar_allreduce(ctx, xd.data_ptr(), o.data_ptr(), n, algo, stream), "rdb_ar_allreduce")
            check(L.rdb_skinny_gemm_fp8_allreduce(ctx, arr, lin.data_ptr(), stream), "rdb_skinny_gemm_fp8_allreduce")

        def verify(x):
            torch.cuda.synchronize()
            assert L.rdb_device_status() == 0
            v1 = oracle.allreduce_fp8(_bits(x)[None])[0]
            assert np.array_equal(_bits(outs[0]), v1) and np.array_equal(_bits(outs[1]), v1)
            assert np.array_equal(_bits(outs[2]), oracle.allreduce_fp8_regather(_bits(x)[None]))
            assert np.array_equal(_bits(lin.reshape(-1)), want_lin)

        x = torch.randn(n, generator=torch.Generator().manual_seed(1)).bfloat16()
        xd.copy_(x)
        issue(torch.cuda.current_stream().cuda_stream)                           # before any capture: per-device set-up
        verify(x)
        assert L.rdb_ar_set_device_epoch(ctx, 0) == 6                            # too late to change the way of counting
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream(device=cuda_device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                issue(side.cuda_stream)
        torch.cuda.current_stream().wait_stream(side)
        for rep in range(5):
            x = torch.randn(n, generator=torch.Generator().manual_seed(10 + rep)).bfloat16() * (rep + 1)
            xd.copy_(x)
            for o in outs:
                o.zero_()
            lin.zero_()
            graph.replay()
            verify(x)
            if rep == 2:                                                          # a direct call between two replays
                check(L.rdb_ar_allreduce(ctx, xd.data_ptr(), outs[0].data_ptr(), n, 2, torch.cuda.current_stream().cuda_stream), "direct")
                verify(x)
        del graph
        L.rdb_ar_destroy(ctx)
        ws.free()


@pytest.mark.gpu
def test_error_codes(cuda_device):
    import ctypes as C
    import rocm_dev_b200 as R
    L = R.lib()
    lr = R.LocalRanks(2, max_elems=4096, device=cuda_device)
    try:
        x = torch.zeros(8192, dtype=torch.bfloat16, device=cuda_device)
        assert L.rdb_ar_allreduce(lr.ctx[0], x.data_ptr(), x.data_ptr(), 100, 0, 0) == 8       # not a multiple of 128
        assert L.rdb_ar_allreduce(lr.ctx[0], x.data_ptr(), x.data_ptr(), 8192, 0, 0) == 11     # above max_elems
        assert L.rdb_ar_allreduce(lr.ctx[0], x.data_ptr() + 2, x.data_ptr(), 128, 0, 0) == 7
        assert L.rdb_ar_allreduce(lr.ctx[0], x.data_ptr(), None, 128, 1, 0) == 6               # one-shot needs out
        assert L.rdb_ar_workspace_bytes(9, 128) == 0
        ctx = C.c_void_p()
        assert L.rdb_ar_create(2, 2, (C.c_void_p * 2)(), 128, C.byref(ctx)) == 6
    finally:
        lr.close()


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 3, 8])
def test_emulated_ranks_deliver_into_registered_buffers(cuda_device, oracle, world):
    """Two-shot calls whose `out` lies in the registered result buffers: every
    rank stores its reduced shard straight into all ranks' buffers (no copy out
    of the workspace); same bits, also at an offset and next to unregistered calls."""
    import rocm_dev_b200 as R
    cap = 1 << 20
    lr = R.LocalRanks(world, max_elems=cap, device=cuda_device)
    try:
        bufs = lr.new_result_buffers(cap)
        for n, off in ((128, 0), (640, 512), (128 * 517, 1024), (cap, 0)):
            for rep in range(2):
                xs = [torch.randn(n, generator=torch.Generator().manual_seed(31 * rep + r + n)).bfloat16() for r in range(world)]
                for b in bufs:
                    b.zero_()
                outs = lr.all_reduce([x.to(cuda_device) for x in xs], algo=2, outs=[b[off:off + n] for b in bufs])
                torch.cuda.synchronize()
                assert R.lib().rdb_device_status() == 0
                want, _, _ = oracle.allreduce_fp8(np.stack([_bits(x) for x in xs]))
                for r in range(world):
                    assert np.array_equal(_bits(outs[r]), want), (world, n, rep, r)
                    assert not bufs[r][:off].any() and not bufs[r][off + n:].any()   # nothing outside the window
                plain = lr.all_reduce([x.to(cuda_device) for x in xs], algo=2)       # ordinary buffers still work
                assert np.array_equal(_bits(plain[0]), want)
    finally:
        lr.close()


@pytest.mark.gpu
@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("M,N,K", [(8, 4096, 4096), (16, 1024, 2048), (3, 384, 512), (32, 6144, 1024), (1, 128, 128)])
def test_gemm_epilogue_feeds_the_allreduce(cuda_device, oracle, world, M, N, K):
    """Row-parallel linear + allreduce with the fused epilogue: K is split over
    the (emulated) ranks, each rank's GEMM quantises its bf16 partial product
    and delivers it to every rank's staging area, the consuming launch reduces.
    Bit-exact against the oracle's allreduce of the partial products that the
    plain grouped GEMM writes for the same slices - which in turn meet the GEMM
    tolerance against the oracle's GEMM."""
    import rocm_dev_b200 as R
    from rocm_dev_b200 import quant
    from helpers import bf16_bits, check_gemm_parity
    if K % (128 * world) != 0:
        pytest.skip("K slice must stay a multiple of 128 bytes")
    dev = cuda_device
    Aq, Bq, sa, sb = quant.synthetic_gemm_operands(M, N, K, seed=world + M)
    kr = K // world
    ops = [(Aq[:, r * kr:(r + 1) * kr].contiguous().to(dev), Bq[:, r * kr:(r + 1) * kr].contiguous().to(dev), sa.to(dev), sb.to(dev))
           for r in range(world)]
    lr = R.LocalRanks(world, max_elems=1 << 20, device=dev)
    try:
        for rep in range(2):                                  # both staging sets
            outs = lr.skinny_gemm_all_reduce(ops)
            torch.cuda.synchronize()
            assert R.lib().rdb_device_status() == 0
            partial = []
            for r, (A, B, a, b) in enumerate(ops):            # the unfused composition, same kernels
                D = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
                assert R.skinny_gemm_fp8_grouped([(A, B, a, b, D)]) == 0
                partial.append(D)
                ref = oracle.gemm_fp8_bf16(A.cpu().numpy(), B.cpu().numpy(), sa.item(), sb.item())
                ref64, mag = oracle.gemm_fp8_f64(A.cpu().numpy(), B.cpu().numpy(), sa.item(), sb.item())
                check_gemm_parity(bf16_bits(D), ref, ref64, mag, kr)
            want, _, _ = oracle.allreduce_fp8(np.stack([_bits(p.reshape(-1)) for p in partial]))
            for r in range(world):
                assert np.array_equal(_bits(outs[r].reshape(-1)), want), (world, M, N, K, rep, r)
            # an ordinary call on the same contexts afterwards (epochs and staging sets stay in step)
            xs = [torch.randn(1024, generator=torch.Generator().manual_seed(r)).bfloat16().to(dev) for r in range(world)]
            got = lr.all_reduce(xs, algo=1)
            w2, _, _ = oracle.allreduce_fp8(np.stack([_bits(x) for x in xs]))
            assert np.array_equal(_bits(got[0]), w2)
    finally:
        lr.close()


@pytest.mark.gpu
def test_fused_linear_rejects_what_it_cannot_do(cuda_device):
    import rocm_dev_b200 as R
    from rocm_dev_b200.skinny_gemm import SkinnyProblem
    import ctypes as C
    L = R.lib()
    lr = R.LocalRanks(1, max_elems=4096, device=cuda_device)
    try:
        x = torch.zeros(1 << 16, dtype=torch.uint8, device=cuda_device)
        f = torch.ones(1, device=cuda_device)
        pr = lambda M, N, K: SkinnyProblem(x.data_ptr(), x.data_ptr(), f.data_ptr(), f.data_ptr(), None, M, N, K, K)  # noqa: E731
        assert L.rdb_skinny_gemm_fp8_allreduce_begin(lr.ctx[0], C.byref(pr(8, 192, 128)), 0) == 8      # N % 128
        assert L.rdb_skinny_gemm_fp8_allreduce_begin(lr.ctx[0], C.byref(pr(32, 256, 128)), 0) == 11    # above max_elems
        assert L.rdb_skinny_gemm_fp8_allreduce_finish(lr.ctx[0], x.data_ptr(), 0) == 6                 # nothing open
        assert L.rdb_skinny_gemm_fp8_allreduce_begin(lr.ctx[0], C.byref(pr(8, 128, 40)), 0) == 3       # refused by the GEMM ...
        out = torch.empty(8 * 128, dtype=torch.bfloat16, device=cuda_device)
        assert L.rdb_ar_allreduce(lr.ctx[0], out.data_ptr(), out.data_ptr(), 1024, 1, 0) == 0          # ... and the epoch was given back
        torch.cuda.synchronize()
        assert L.rdb_device_status() == 0
    finally:
        lr.close()


@pytest.mark.gpu
def test_a_wait_that_runs_out_is_reported_and_leaves_everything_usable(cuda_device, oracle):
    """Failure detection without a fault: with a 2 ms wait budget, rank 0's
    reduce step is issued while rank 1's encoded blocks are withheld by the
    host.  The wait gives up by construction: the kernel returns, the status
    word says RDB_DEVICE_TIMEOUT, rank 0 publishes its delivery flag marked
    failed, and rank 1 - which does everything right, only late - sees that mark
    and reports the failure as well instead of copying a shard that was never
    written.  With the budget restored the same contexts then give bit-exact
    results (both staging sets)."""
    import rocm_dev_b200 as R
    from rocm_dev_b200._lib import check
    L = R.lib()
    n = 128 * 64
    lr = R.LocalRanks(2, max_elems=1 << 16, device=cuda_device)
    try:
        xs = [torch.randn(n, generator=torch.Generator().manual_seed(r)).bfloat16().to(cuda_device) for r in range(2)]
        outs = [torch.zeros(n, dtype=torch.bfloat16, device=cuda_device) for _ in range(2)]
        stream = torch.cuda.current_stream().cuda_stream
        with torch.cuda.device(cuda_device):
            assert L.rdb_set_wait_budget_ns(2_000_000) == 0
            try:
                epoch = {int(L.rdb_ar_begin_call(c)) for c in lr.ctx}.pop()
                args = lambda r: (xs[r].data_ptr(), outs[r].data_ptr(), n, 2, stream)   # noqa: E731
                check(L.rdb_ar_phase(lr.ctx[0], 1, epoch, *args(0)), "push 0")
                check(L.rdb_ar_phase(lr.ctx[0], 2, epoch, *args(0)), "reduce 0")       # rank 1 has not pushed
                torch.cuda.synchronize()
                assert L.rdb_device_status() == 10                                      # reported, kernel returned
                assert L.rdb_device_status() == 0                                       # reading clears it
                check(L.rdb_ar_phase(lr.ctx[1], 1, epoch, *args(1)), "push 1")
                check(L.rdb_ar_phase(lr.ctx[1], 2, epoch, *args(1)), "reduce 1")
                check(L.rdb_ar_phase(lr.ctx[1], 3, epoch, *args(1)), "gather 1")
                check(L.rdb_ar_phase(lr.ctx[0], 3, epoch, *args(0)), "gather 0")
                torch.cuda.synchronize()
                assert L.rdb_device_status() == 10                                      # rank 0's failure mark was seen
                assert not outs[1].any() and not outs[0].any()                          # nobody copied a partial result
            finally:
                assert L.rdb_set_wait_budget_ns(1_000_000_000) == 0
        # the same for the one-shot transport, whose receivers poll the data lines themselves: rank 0 reduces while
        # rank 1's lines are missing -> its wait gives up, reports, and writes nothing for the groups it could not finish
        with torch.cuda.device(cuda_device):
            assert L.rdb_set_wait_budget_ns(2_000_000) == 0
            try:
                epoch = {int(L.rdb_ar_begin_call(c)) for c in lr.ctx}.pop()
                outs[0].zero_()
                args1 = lambda r: (xs[r].data_ptr(), outs[r].data_ptr(), n, 1, stream)   # noqa: E731
                check(L.rdb_ar_phase(lr.ctx[0], 1, epoch, *args1(0)), "ll push 0")
                check(L.rdb_ar_phase(lr.ctx[0], 2, epoch, *args1(0)), "ll reduce 0")
                torch.cuda.synchronize()
                assert L.rdb_device_status() == 10 and not outs[0].any()
                check(L.rdb_ar_phase(lr.ctx[1], 1, epoch, *args1(1)), "ll push 1")      # the late rank still completes
                check(L.rdb_ar_phase(lr.ctx[1], 2, epoch, *args1(1)), "ll reduce 1")
                torch.cuda.synchronize()
                assert L.rdb_device_status() == 0
                want1, _, _ = oracle.allreduce_fp8(np.stack([_bits(x) for x in xs]))
                assert np.array_equal(_bits(outs[1]), want1)
            finally:
                assert L.rdb_set_wait_budget_ns(1_000_000_000) == 0
        for rep in range(2):                                                            # GPU and contexts are reusable
            got = lr.all_reduce(xs, algo=1)
            torch.cuda.synchronize()
            assert L.rdb_device_status() == 0
            want, _, _ = oracle.allreduce_fp8(np.stack([_bits(x) for x in xs]))
            assert np.array_equal(_bits(got[0]), want) and np.array_equal(_bits(got[1]), want)
        for rep in range(2):
            got = lr.all_reduce(xs, algo=2)
            torch.cuda.synchronize()
            assert L.rdb_device_status() == 0
            want, _, _ = oracle.allreduce_fp8(np.stack([_bits(x) for x in xs]))
            assert np.array_equal(_bits(got[0]), want) and np.array_equal(_bits(got[1]), want)
    finally:
        lr.close()


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("backend", ["ipc", "symm"])
def test_one_process_per_gpu(cuda_device, backend, world):
    """Real peer-to-peer path: one process per GPU; workspaces shared by CUDA
    IPC, or allocated as symmetric memory (multimem all-gather where the
    allocation has a multicast address)."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1",
               MASTER_PORT=str(29600 + os.getpid() % 300 + (7 if backend == "symm" else 0) + world),
               WORLD_SIZE=str(world), RDB_AR_BACKEND=backend)
    procs = [subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "ar_worker.py")], env=dict(env, RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = [p.communicate(timeout=600)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)
    assert all(f"rank {r} ok" in outs[r] for r in range(world))
