"""GPU parity tests of the skinny FP8 GEMM against the CPU oracle, through the
C ABI.  Tolerance: relative Frobenius error <= 1e-2 and <= 2 bf16 ulp per
element (see helpers.check_gemm_parity for the fp64 adjudication rule)."""
import json
import os

import numpy as np
import pytest
import torch

from helpers import bf16_bits, check_gemm_parity

pytestmark = pytest.mark.gpu


def _run(dev, Aq, Bq, sa, sb, **kw):
    import rocm_dev_b200 as R
    out = R.skinny_gemm_fp8(Aq.to(dev), Bq.to(dev), sa.to(dev), sb.to(dev), **kw)
    torch.cuda.synchronize()
    assert R.lib().rdb_device_status() == 0
    return out


def _parity(oracle, dev, M, N, K, seed=0):
    from rocm_dev_b200 import quant
    Aq, Bq, sa, sb = quant.synthetic_gemm_operands(M, N, K, seed=seed)
    out = _run(dev, Aq, Bq, sa, sb)
    ref = oracle.gemm_fp8_bf16(Aq.numpy(), Bq.numpy(), sa.item(), sb.item())
    ref64, mag = oracle.gemm_fp8_f64(Aq.numpy(), Bq.numpy(), sa.item(), sb.item())
    return check_gemm_parity(bf16_bits(out), ref, ref64, mag, K)


def test_tiny_known_answer(cuda_device):
    with open(os.path.join(os.path.dirname(__file__), "golden", "known_answers.json")) as f:
        t = json.load(f)["tiny_gemm"]
    A = torch.tensor(t["A"], dtype=torch.uint8)
    B = torch.tensor(t["B"], dtype=torch.uint8)
    out = _run(cuda_device, A, B, torch.tensor([t["scale_a"]]), torch.tensor([t["scale_b"]]))
    assert bf16_bits(out).tolist() == t["D_bf16"]


def test_one_hot_rows_select_weight_columns(cuda_device, oracle):
    """The reference's commented probe: a one-hot activation row picks one
    column of the weights, exactly."""
    N, K = 256, 512
    g = torch.Generator().manual_seed(2)
    B = torch.randint(0, 0x7E, (N, K), generator=g, dtype=torch.uint8)
    A = torch.zeros((4, K), dtype=torch.uint8)
    cols = [0, 127, 128, 511]
    for i, c in enumerate(cols):
        A[i, c] = 0x38
    one = torch.ones(1)
    out = _run(cuda_device, A, B, one, one)
    want = oracle.bf16_encode(oracle.e4m3fn_decode(B.numpy()[:, cols].T.copy()))
    assert np.array_equal(bf16_bits(out), want)


@pytest.mark.parametrize("M", [1, 2, 4, 8, 16, 32])
def test_config0_shape_all_m(cuda_device, oracle, M):
    r = _parity(oracle, cuda_device, M, 8192, 8192)
    assert r["rel_fro"] < 1e-2


@pytest.mark.parametrize("N,K", [(6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336)])
@pytest.mark.parametrize("M", [1, 2, 4, 8, 16, 32])
def test_decode_sweep_shapes(cuda_device, oracle, M, N, K):
    _parity(oracle, cuda_device, M, N, K, seed=M)


@pytest.mark.parametrize("M,N,K", [(3, 130, 144), (7, 2, 16), (17, 1000, 272), (32, 258, 4112), (5, 126, 128),
                                   (9, 384, 48), (1, 64, 8192)])
def test_ragged_edges(cuda_device, oracle, M, N, K):
    _parity(oracle, cuda_device, M, N, K, seed=4)


@pytest.mark.parametrize("split_k", [1, 2, 3, 4, 5, 7, 8])
def test_every_cluster_size_gives_the_same_answer(cuda_device, oracle, split_k):
    import rocm_dev_b200 as R
    from rocm_dev_b200 import quant
    M, N, K = 8, 512, 2048
    Aq, Bq, sa, sb = quant.synthetic_gemm_operands(M, N, K, seed=6)
    dev = cuda_device
    dA, dB, dsa, dsb = Aq.to(dev), Bq.to(dev), sa.to(dev), sb.to(dev)
    D = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    code = R.skinny_gemm(dA, dB, D, dsa, M, N, K, K, split_k, 1, 1, 1, 1, 4, 8, 2)
    assert code == 0
    torch.cuda.synchronize()
    assert R.lib().rdb_device_status() == 0
    # scale_b is 1 in the reference-named launcher
    ref = oracle.gemm_fp8_bf16(Aq.numpy(), Bq.numpy(), sa.item(), 1.0)
    ref64, mag = oracle.gemm_fp8_f64(Aq.numpy(), Bq.numpy(), sa.item(), 1.0)
    check_gemm_parity(bf16_bits(D), ref, ref64, mag, K)


# ------------------------------------------------------------ grouped entry
def _grouped(oracle, dev, shapes, seed=0, pitch=None):
    """Runs `shapes` = [(M, N, K), ...] as ONE grouped launch and checks every
    problem against the oracle with the stated tolerance."""
    import rocm_dev_b200 as R
    from rocm_dev_b200 import quant
    host, problems = [], []
    for i, (M, N, K) in enumerate(shapes):
        Aq, Bq, sa, sb = quant.synthetic_gemm_operands(M, N, K, seed=seed + i)
        host.append((Aq, Bq, sa, sb))
        dB = Bq.to(dev)
        if pitch:                                   # weights inside a wider allocation: row pitch > K
            wide = torch.full((N, K + pitch), 0x7E, dtype=torch.uint8, device=dev)
            wide[:, :K] = dB
            dB = wide[:, :K]
        D = torch.full((M, N), 77.0, dtype=torch.bfloat16, device=dev)      # overwritten, not accumulated into
        problems.append((Aq.to(dev), dB, sa.to(dev), sb.to(dev), D))
    assert R.skinny_gemm_fp8_grouped(problems) == 0
    torch.cuda.synchronize()
    assert R.lib().rdb_device_status() == 0
    reports = []
    for (M, N, K), (Aq, Bq, sa, sb), pr in zip(shapes, host, problems):
        ref = oracle.gemm_fp8_bf16(Aq.numpy(), Bq.numpy(), sa.item(), sb.item())
        ref64, mag = oracle.gemm_fp8_f64(Aq.numpy(), Bq.numpy(), sa.item(), sb.item())
        reports.append(check_gemm_parity(bf16_bits(pr[4]), ref, ref64, mag, K))
    return problems, reports


def test_grouped_tiny_and_ragged_problems(cuda_device, oracle):
    """Fewer units than CTAs (most CTAs idle, tiles shared by single-unit
    ranges), ragged M / N / K, both activation paddings."""
    _grouped(oracle, cuda_device, [(8, 64, 256), (3, 48, 144)])
    _grouped(oracle, cuda_device, [(3, 130, 144), (7, 2, 16), (17, 1000, 272), (32, 258, 4112), (5, 126, 128),
                                   (9, 384, 48), (1, 64, 8192)], seed=4)
    _grouped(oracle, cuda_device, [(4, 300, 2048)], seed=9, pitch=256)


@pytest.mark.parametrize("M", [1, 8, 32])
def test_grouped_config0_shape(cuda_device, oracle, M):
    """Config 0 (N = K = 8192) as a single-problem list: 128-row units, every tile shared by several CTAs."""
    _, rep = _grouped(oracle, cuda_device, [(M, 8192, 8192)])
    assert rep[0]["rel_fro"] < 1e-2


@pytest.mark.parametrize("M", [1, 2, 4, 8, 16])
def test_grouped_decode_layer(cuda_device, oracle, M):
    """The four projections of one decode layer at one M, one launch."""
    _grouped(oracle, cuda_device, [(M, 6144, 4096), (M, 4096, 4096), (M, 28672, 4096), (M, 4096, 14336)], seed=M)


def test_grouped_whole_sweep_is_deterministic_and_replayable(cuda_device, oracle):
    """All 20 (shape, M) cases of the decode sweep in one launch: parity for
    every problem, identical bits when launched again and when replayed from a
    CUDA graph (the launch keeps no state that a replay could see stale)."""
    import rocm_dev_b200 as R
    shapes = [(M, N, K) for M in (1, 2, 4, 8, 16) for (N, K) in ((6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336))]
    problems, _ = _grouped(oracle, cuda_device, shapes, seed=50)
    first = [p[4].clone() for p in problems]
    for p in problems:
        p[4].zero_()
    assert R.skinny_gemm_fp8_grouped(problems) == 0
    torch.cuda.synchronize()
    assert all(torch.equal(a, p[4]) for a, p in zip(first, problems))
    stream = torch.cuda.Stream(device=cuda_device)
    with torch.cuda.stream(stream):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            assert R.skinny_gemm_fp8_grouped(problems) == 0
        for _ in range(3):
            for p in problems:
                p[4].zero_()
            g.replay()
            g.replay()
            torch.cuda.synchronize()
            assert all(torch.equal(a, p[4]) for a, p in zip(first, problems))
    assert R.lib().rdb_device_status() == 0
    # programmatic launch: each launch streams weights while the one before drains; four in a row, with a plain
    # per-GEMM launch in between, leave the same bits
    for p in problems:
        p[4].zero_()
    for i in range(4):
        assert R.skinny_gemm_fp8_grouped(problems, flags=R.OVERLAP_PRIOR_KERNEL) == 0
        if i == 1:
            R.skinny_gemm_fp8(problems[0][0], problems[0][1], problems[0][2], problems[0][3])
    torch.cuda.synchronize()
    assert R.lib().rdb_device_status() == 0
    assert all(torch.equal(a, p[4]) for a, p in zip(first, problems))
    with torch.cuda.stream(stream):
        g2 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g2, stream=stream):
            for _ in range(3):             # the same list each time: the K split, and so the bits, depend on the list
                assert R.skinny_gemm_fp8_grouped(problems, flags=R.OVERLAP_PRIOR_KERNEL) == 0
        for p in problems:
            p[4].zero_()
        g2.replay()
        g2.replay()
        torch.cuda.synchronize()
    assert all(torch.equal(a, p[4]) for a, p in zip(first, problems))
    assert R.lib().rdb_device_status() == 0
    assert R.lib().rdb_skinny_gemm_fp8_grouped(None, 1, 2, 0) == 6          # unknown flag


def test_grouped_matches_the_plan_and_rejects_bad_lists(cuda_device):
    import ctypes as C
    import rocm_dev_b200 as R
    from rocm_dev_b200.skinny_gemm import SkinnyProblem
    rows, ranges = R.skinny_gemm_grouped_plan([(8, 6144, 4096), (8, 4096, 14336)], ctas=148)
    assert rows == [256, 256] and ranges[0] == 0 and ranges[-1] == 24 * 32 + 16 * 112
    assert all(b >= a for a, b in zip(ranges, ranges[1:])) and max(b - a for a, b in zip(ranges, ranges[1:])) <= 18
    L = R.lib()
    x = torch.zeros(4096, dtype=torch.uint8, device=cuda_device)
    f = torch.ones(1, device=cuda_device)
    ok = SkinnyProblem(x.data_ptr(), x.data_ptr(), f.data_ptr(), f.data_ptr(), x.data_ptr(), 8, 16, 64, 64)
    assert L.rdb_skinny_gemm_fp8_grouped(C.byref(ok), 0, 0, 0) == 6
    assert L.rdb_skinny_gemm_fp8_grouped(C.byref(ok), 33, 0, 0) == 6
    bad = SkinnyProblem(x.data_ptr(), x.data_ptr(), f.data_ptr(), f.data_ptr(), x.data_ptr(), 33, 16, 64, 64)
    assert L.rdb_skinny_gemm_fp8_grouped(C.byref(bad), 1, 0, 0) == 1
    bad = SkinnyProblem(x.data_ptr(), x.data_ptr(), f.data_ptr(), f.data_ptr(), x.data_ptr(), 8, 15, 64, 64)
    assert L.rdb_skinny_gemm_fp8_grouped(C.byref(bad), 1, 0, 0) == 2
    bad = SkinnyProblem(x.data_ptr(), x.data_ptr(), f.data_ptr(), f.data_ptr(), x.data_ptr(), 8, 16, 40, 48)
    assert L.rdb_skinny_gemm_fp8_grouped(C.byref(bad), 1, 0, 0) == 3
    bad = SkinnyProblem(x.data_ptr() + 1, x.data_ptr(), f.data_ptr(), f.data_ptr(), x.data_ptr(), 8, 16, 64, 64)
    assert L.rdb_skinny_gemm_fp8_grouped(C.byref(bad), 1, 0, 0) == 7


def test_row_pitch_and_output_overwrite(cuda_device, oracle):
    """B with a row pitch larger than K, and D pre-filled with garbage: the
    result is overwritten, not accumulated into."""
    import rocm_dev_b200 as R
    from rocm_dev_b200 import quant
    M, N, K, ld = 8, 256, 1024, 1280
    Aq, Bq, sa, sb = quant.synthetic_gemm_operands(M, N, K, seed=8)
    dev = cuda_device
    Bp = torch.full((N, ld), 0x7E, dtype=torch.uint8, device=dev)
    Bp[:, :K] = Bq.to(dev)
    D = torch.full((M, N), 123.0, dtype=torch.bfloat16, device=dev)
    R.skinny_gemm_fp8(Aq.to(dev), Bp[:, :K], sa.to(dev), sb.to(dev), out=D)
    ref = oracle.gemm_fp8_bf16(Aq.numpy(), Bq.numpy(), sa.item(), sb.item())
    ref64, mag = oracle.gemm_fp8_f64(Aq.numpy(), Bq.numpy(), sa.item(), sb.item())
    check_gemm_parity(bf16_bits(D), ref, ref64, mag, K)


def test_deterministic_across_runs(cuda_device):
    from rocm_dev_b200 import quant
    Aq, Bq, sa, sb = quant.synthetic_gemm_operands(16, 4096, 4096, seed=1)
    dev = cuda_device
    args = (Aq.to(dev), Bq.to(dev), sa.to(dev), sb.to(dev))
    import rocm_dev_b200 as R
    first = R.skinny_gemm_fp8(*args).clone()
    for _ in range(20):
        assert torch.equal(R.skinny_gemm_fp8(*args), first)


def test_linearity_in_scale(cuda_device):
    """Doubling scale_a doubles every output exactly (power-of-two scaling)."""
    from rocm_dev_b200 import quant
    import rocm_dev_b200 as R
    Aq, Bq, sa, sb = quant.synthetic_gemm_operands(4, 1024, 1024, seed=3)
    dev = cuda_device
    d1 = R.skinny_gemm_fp8(Aq.to(dev), Bq.to(dev), sa.to(dev), sb.to(dev)).float()
    d2 = R.skinny_gemm_fp8(Aq.to(dev), Bq.to(dev), (2 * sa).to(dev), sb.to(dev)).float()
    assert torch.equal(d2, 2 * d1)


def test_error_codes(cuda_device):
    import rocm_dev_b200 as R
    from rocm_dev_b200 import SkinnyGemmReturnCode as C
    dev = cuda_device
    A = torch.zeros((8, 256), dtype=torch.uint8, device=dev)
    B = torch.zeros((64, 256), dtype=torch.uint8, device=dev)
    D = torch.zeros((8, 64), dtype=torch.bfloat16, device=dev)
    s = torch.ones(1, device=dev)
    assert R.skinny_gemm_fastpath(A, B, D, s, 8, 63, 256) == C.N_NOT_EVEN
    assert R.skinny_gemm_fastpath(A, B, D, s, 8, 64, 250) == C.K_NOT_DIVISIBLE_BY_WARPTILE_K
    assert R.skinny_gemm_fastpath(A, B, D, s, 33, 64, 256) == C.M_ABOVE_WARPTILE_M
    assert R.skinny_gemm_fastpath(A, B, D, s, 0, 64, 256) == C.BAD_SHAPE
    assert R.skinny_gemm_fastpath(A.data_ptr() + 1, B, D, s, 8, 64, 256) == C.BAD_ALIGNMENT
    # reference validation of the tuning arguments
    assert R.skinny_gemm(A, B, D, s, 8, 64, 256, 256, 1, 8, 8, 8, 1, 8, 8, 2) == C.TOO_MANY_WARPS
    assert R.skinny_gemm(A, B, D, s, 8, 64, 256, 256, 1, 2, 2, 2, 1, 1, 8, 2) == C.QSIZE_TOO_SMALL
    assert R.skinny_gemm(A, B, D, s, 8, 64, 256, 256, 1, 1, 1, 1, 0, 1, 8, 2) == C.INVALID_CONFIG
    assert R.skinny_gemm(A, B, D, s, 8, 64, 192, 256, 1, 1, 1, 1, 1, 1, 8, 2) == C.K_NOT_DIVISIBLE_BY_WARPTILE_K
    assert R.skinny_gemm_fastpath(A, B, D, s, 8, 64, 256) == C.SUCCESS
    torch.cuda.synchronize()


def test_torch_binding_mirror(cuda_device, oracle):
    """HFRK_skinny_gemm: B passed as the [K,N] view of [N,K] storage."""
    import rocm_dev_b200 as R
    from rocm_dev_b200 import quant
    M, N, K = 16, 512, 1024
    Aq, Bq, sa, sb = quant.synthetic_gemm_operands(M, N, K, seed=12)
    dev = cuda_device
    D = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    import hfrk_skinny_gemm                      # the module name callers of the reference import
    assert hfrk_skinny_gemm.HFRK_skinny_gemm is R.HFRK_skinny_gemm
    h = hfrk_skinny_gemm.HFRK_skinny_gemm(1)
    code = h.skinny_gemm_torch_binding(Aq.to(dev).view(torch.float8_e4m3fn), Bq.to(dev).view(torch.float8_e4m3fn).t(),
                                       D, sa.to(dev), 2, 1, 1, 1, 1, 4, 2)
    assert code == 0
    ref = oracle.gemm_fp8_bf16(Aq.numpy(), Bq.numpy(), sa.item(), 1.0)
    ref64, mag = oracle.gemm_fp8_f64(Aq.numpy(), Bq.numpy(), sa.item(), 1.0)
    check_gemm_parity(bf16_bits(D), ref, ref64, mag, K)


def test_host_buffer_entry(cuda_device, oracle):
    import rocm_dev_b200 as R
    from rocm_dev_b200 import quant
    M, N, K = 8, 1024, 1024
    Aq, Bq, sa, sb = quant.synthetic_gemm_operands(M, N, K, seed=13)
    out = torch.empty((M, N), dtype=torch.bfloat16).pin_memory()
    R.skinny_gemm_fp8_host(Aq.pin_memory(), Bq.pin_memory(), sa.pin_memory(), sb.pin_memory(), out)
    ref = oracle.gemm_fp8_bf16(Aq.numpy(), Bq.numpy(), sa.item(), sb.item())
    ref64, mag = oracle.gemm_fp8_f64(Aq.numpy(), Bq.numpy(), sa.item(), sb.item())
    check_gemm_parity(bf16_bits(out), ref, ref64, mag, K)
