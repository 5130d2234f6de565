"""GPU parity tests of the dense FP8 GEMM (the async_gemm projects) against the
CPU oracle, through the C ABI.  bf16 path: relative Frobenius <= 1e-2 and <= 2
bf16 ulp per element (fp64 adjudication as in helpers.check_gemm_parity).
fp32 path (the reference's unscaled output): |got - fp64| <= 4*sqrt(K)*2^-24 *
sum|a*b| per element, the summation-order noise of an fp32 accumulation."""
import numpy as np
import pytest
import torch

from helpers import bf16_bits, check_gemm_parity

pytestmark = pytest.mark.gpu


def _operands(M, N, K, seed, w_std=1.0):
    from rocm_dev_b200 import quant
    return quant.synthetic_gemm_operands(M, N, K, seed=seed, w_std=w_std)


def _check_bf16(oracle, dev, M, N, K, seed=0):
    import rocm_dev_b200 as R
    Aq, Bq, sa, sb = _operands(M, N, K, seed)
    out = R.dense_gemm_fp8(Aq.to(dev), Bq.to(dev), sa.to(dev), sb.to(dev))
    torch.cuda.synchronize()
    assert R.lib().rdb_device_status() == 0
    ref = oracle.gemm_fp8_bf16(Aq.numpy(), Bq.numpy(), sa.item(), sb.item())
    ref64, mag = oracle.gemm_fp8_f64(Aq.numpy(), Bq.numpy(), sa.item(), sb.item())
    return check_gemm_parity(bf16_bits(out), ref, ref64, mag, K)


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (128, 256, 512), (256, 512, 1024), (384, 768, 2048),
                                   (1024, 1024, 1024)])
def test_tile_multiples(cuda_device, oracle, M, N, K):
    _check_bf16(oracle, cuda_device, M, N, K)


@pytest.mark.parametrize("M,N,K", [(1, 8, 16), (100, 200, 144), (130, 258, 272), (129, 1000, 4112), (16, 48, 64),
                                   (8, 64, 64), (300, 40, 1024)])
def test_ragged_shapes(cuda_device, oracle, M, N, K):
    _check_bf16(oracle, cuda_device, M, N, K, seed=3)


@pytest.mark.parametrize("tile_rows", [128, 256])
@pytest.mark.parametrize("M,N,K", [(512, 512, 1024), (300, 520, 272), (1280, 768, 512)])
def test_both_tile_heights(cuda_device, oracle, tile_rows, M, N, K):
    import rocm_dev_b200 as R
    Aq, Bq, sa, sb = _operands(M, N, K, seed=11)
    dev = cuda_device
    out = R.dense_gemm_fp8(Aq.to(dev), Bq.to(dev), sa.to(dev), sb.to(dev), tile_rows=tile_rows, max_ctas=3)
    torch.cuda.synchronize()
    assert R.lib().rdb_device_status() == 0
    ref = oracle.gemm_fp8_bf16(Aq.numpy(), Bq.numpy(), sa.item(), sb.item())
    ref64, mag = oracle.gemm_fp8_f64(Aq.numpy(), Bq.numpy(), sa.item(), sb.item())
    check_gemm_parity(bf16_bits(out), ref, ref64, mag, K)


@pytest.mark.parametrize("M,N,K", [(512, 512, 1024), (300, 520, 384), (1280, 768, 512), (257, 255, 128), (512, 256, 896)])
def test_cta_pairs_with_three_k_blocks_per_stage(cuda_device, M, N, K):
    """tile_rows = 3: same tiles, deeper stages (K not a multiple of 384 ends in a zero-filled chunk); the
    accumulation order is unchanged, so the bits equal the two-chunk pair kernel's."""
    import rocm_dev_b200 as R
    Aq, Bq, sa, sb = _operands(M, N, K, seed=17)
    dev = cuda_device
    a = R.dense_gemm_fp8(Aq.to(dev), Bq.to(dev), sa.to(dev), sb.to(dev), tile_rows=3)
    b = R.dense_gemm_fp8(Aq.to(dev), Bq.to(dev), sa.to(dev), sb.to(dev), tile_rows=2)
    torch.cuda.synchronize()
    assert R.lib().rdb_device_status() == 0
    assert torch.equal(a, b)


@pytest.mark.parametrize("max_ctas", [2, 0])
@pytest.mark.parametrize("M,N,K", [(512, 512, 1024), (300, 520, 384), (1280, 768, 512), (257, 255, 128), (100, 40, 256)])
def test_cta_pairs(cuda_device, oracle, max_ctas, M, N, K):
    """256 x 256 tiles computed by pairs of CTAs (forced: the automatic choice skips shapes with this much
    padding); max_ctas=2 makes a single pair walk every tile, alternating both accumulators."""
    import rocm_dev_b200 as R
    Aq, Bq, sa, sb = _operands(M, N, K, seed=13)
    dev = cuda_device
    out = R.dense_gemm_fp8(Aq.to(dev), Bq.to(dev), sa.to(dev), sb.to(dev), tile_rows=2, max_ctas=max_ctas)
    torch.cuda.synchronize()
    assert R.lib().rdb_device_status() == 0
    ref = oracle.gemm_fp8_bf16(Aq.numpy(), Bq.numpy(), sa.item(), sb.item())
    ref64, mag = oracle.gemm_fp8_f64(Aq.numpy(), Bq.numpy(), sa.item(), sb.item())
    check_gemm_parity(bf16_bits(out), ref, ref64, mag, K)
    # the pair kernel and the single-CTA kernel accumulate in the same order: identical bits
    single = R.dense_gemm_fp8(Aq.to(dev), Bq.to(dev), sa.to(dev), sb.to(dev), tile_rows=128)
    assert torch.equal(out, single)


def test_cta_pairs_reject_k_not_multiple_of_128(cuda_device):
    import rocm_dev_b200 as R
    dev = cuda_device
    A = torch.zeros((256, 272), dtype=torch.uint8, device=dev)
    one = torch.ones(1, device=dev)
    with pytest.raises(Exception):
        R.dense_gemm_fp8(A, A, one, one, tile_rows=2)


def test_many_tiles_per_cta_and_both_accumulators(cuda_device, oracle):
    # 40 x 12 = 480 tiles on 148 CTAs: every CTA runs 3-4 tiles, alternating accumulators
    _check_bf16(oracle, cuda_device, 5120, 3072, 256, seed=5)


def test_config2_smallest_size_sampled(cuda_device, oracle):
    """4096^3 (BASELINE config 2): the oracle checks a sample of rows of A."""
    import rocm_dev_b200 as R
    M = N = K = 4096
    Aq, Bq, sa, sb = _operands(M, N, K, seed=0)
    dev = cuda_device
    out = R.dense_gemm_fp8(Aq.to(dev), Bq.to(dev), sa.to(dev), sb.to(dev))
    rows = np.r_[0:4, 127:131, 2048:2050, 4092:4096]
    ref = oracle.gemm_fp8_bf16(Aq.numpy()[rows], Bq.numpy(), sa.item(), sb.item())
    ref64, mag = oracle.gemm_fp8_f64(Aq.numpy()[rows], Bq.numpy(), sa.item(), sb.item())
    check_gemm_parity(bf16_bits(out[torch.from_numpy(rows).to(dev)]), ref, ref64, mag, K)


def _config2_operands(n, dev, seed, rows=None):
    """A, B ~ N(0,1) quantised per tensor (config 2), drawn and quantised on the GPU."""
    from rocm_dev_b200 import quant
    g = torch.Generator(device=dev).manual_seed(seed)
    Aq, sa = quant.quantize_per_tensor(torch.randn((n if rows is None else rows, n), generator=g, device=dev).bfloat16())
    Bq, sb = quant.quantize_per_tensor(torch.randn((n, n), generator=g, device=dev).bfloat16())
    return Aq, Bq, sa, sb


@pytest.mark.parametrize("n", [8192, 16384])
def test_config2_larger_sizes_sampled(cuda_device, oracle, n):
    """8192^3 and 16384^3 (config 2) through the automatic tiling - the CTA-pair kernel:
    the oracle checks sixteen rows spread over first / interior / last tiles and both CTAs of a pair."""
    import rocm_dev_b200 as R
    dev = cuda_device
    Aq, Bq, sa, sb = _config2_operands(n, dev, seed=n)
    out = R.dense_gemm_fp8(Aq, Bq, sa, sb)
    torch.cuda.synchronize()
    assert R.lib().rdb_device_status() == 0
    rows = np.r_[0:2, 127:130, 255:258, n // 2 - 1:n // 2 + 2, n - 130:n - 128, n - 3:n]
    Bh = Bq.cpu().numpy()
    Ah = Aq[torch.from_numpy(rows).to(dev)].cpu().numpy()
    ref = oracle.gemm_fp8_bf16(Ah, Bh, sa.item(), sb.item())
    ref64, mag = oracle.gemm_fp8_f64(Ah, Bh, sa.item(), sb.item())
    check_gemm_parity(bf16_bits(out[torch.from_numpy(rows).to(dev)]), ref, ref64, mag, n)


def test_rows_sharded_over_two_gpus(cuda_device, oracle):
    """Config 2's multi-GPU form: the M rows of A and D are split over the GPUs, B is replicated, nothing is
    communicated.  Each GPU's rows are checked against the oracle on its rows of A."""
    import rocm_dev_b200 as R
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    n, world = 4096, 2
    Aq, Bq, sa, sb = _config2_operands(n, cuda_device, seed=77)
    Bh = Bq.cpu().numpy()
    for r in range(world):
        dev = torch.device("cuda", r)
        lo, hi = r * n // world, (r + 1) * n // world
        with torch.cuda.device(dev):
            out = R.dense_gemm_fp8(Aq[lo:hi].to(dev).contiguous(), Bq.to(dev), sa.to(dev), sb.to(dev))
            torch.cuda.synchronize(dev)
            assert R.lib().rdb_device_status() == 0
        rows = np.r_[0:3, 255:258, hi - lo - 3:hi - lo]
        Ah = Aq[lo:hi][torch.from_numpy(rows).to(cuda_device)].cpu().numpy()
        ref = oracle.gemm_fp8_bf16(Ah, Bh, sa.item(), sb.item())
        ref64, mag = oracle.gemm_fp8_f64(Ah, Bh, sa.item(), sb.item())
        check_gemm_parity(bf16_bits(out[torch.from_numpy(rows).to(dev)]), ref, ref64, mag, n)


def test_fp32_output_at_a_4_byte_aligned_address(cuda_device, oracle):
    """A D that is only 4-byte aligned (a view into a larger buffer) takes scalar stores; both kernels."""
    import rocm_dev_b200 as R
    dev = cuda_device
    m, n, k = 256, 512, 256
    g = torch.Generator().manual_seed(21)
    A = torch.randint(0, 0x60, (m, k), generator=g, dtype=torch.uint8)
    B = torch.randint(0, 0x60, (n, k), generator=g, dtype=torch.uint8)
    ref32 = oracle.gemm_fp8_f32(A.numpy(), B.numpy())
    ref64, mag = oracle.gemm_fp8_f64(A.numpy(), B.numpy(), 1.0, 1.0)
    tol = 4 * np.sqrt(k) * 2.0 ** -24 * mag + 1e-30
    dA, dB = A.to(dev), B.to(dev)
    for off in (1, 2, 3):
        buf = torch.full((m * n + 4,), -7.0, dtype=torch.float32, device=dev)
        D = buf[off:off + m * n]
        assert R.lib().rdb_dense_gemm_fp8_f32(dA.data_ptr(), dB.data_ptr(), D.data_ptr(), m, n, k, 0) == 0
        torch.cuda.synchronize()
        assert R.lib().rdb_device_status() == 0
        got = D.cpu().numpy().reshape(m, n).astype(np.float64)
        assert (np.abs(got - ref64) <= tol).all()
        assert (buf[:off] == -7.0).all() and (buf[off + m * n:] == -7.0).all()      # nothing outside D
    assert ref32.shape == (m, n)


def test_full_size_properties(cuda_device):
    """8192^3: size-independent properties - a power-of-two scale commutes
    exactly, the product with an identity-like B copies A's values, and two runs
    agree bit for bit."""
    import rocm_dev_b200 as R
    dev = cuda_device
    M = N = K = 8192
    g = torch.Generator(device=dev).manual_seed(1)
    A = torch.randint(0, 0x78, (M, K), generator=g, dtype=torch.uint8, device=dev)
    eye = torch.zeros((N, K), dtype=torch.uint8, device=dev)
    eye[torch.arange(N, device=dev), torch.arange(N, device=dev)] = 0x38      # 1.0
    one = torch.ones(1, device=dev)
    d1 = R.dense_gemm_fp8(A, eye, one, one)
    assert torch.equal(d1.float(), A.view(torch.float8_e4m3fn).float())        # exact: e4m3 fits in bf16
    d2 = R.dense_gemm_fp8(A, eye, 4 * one, one)
    assert torch.equal(d2.float(), 4 * d1.float())
    B = torch.randint(0, 0x78, (N, K), generator=g, dtype=torch.uint8, device=dev)
    x = R.dense_gemm_fp8(A, B, one, one).clone()
    y = R.dense_gemm_fp8(A, B, one, one)
    assert torch.equal(x, y)
    assert R.lib().rdb_device_status() == 0


@pytest.mark.parametrize("project,m,n,k", [("async_gemm_16x16x64", 64, 48, 128), ("async_gemm_blanes", 32, 96, 192),
                                           ("async_gemm_sparse", 8, 64, 64), ("async_gemm_16x16x64", 512, 512, 512)])
def test_reference_named_launcher_fp32(cuda_device, oracle, project, m, n, k):
    import rocm_dev_b200 as R
    g = torch.Generator().manual_seed(2)
    # the reference drivers draw fp8(uniform[-1,1)) without a quantisation step
    A = ((torch.rand((m, k), generator=g) * 2 - 1).clamp(-448, 448)).to(torch.float8_e4m3fn).view(torch.uint8)
    B = ((torch.rand((n, k), generator=g) * 2 - 1).clamp(-448, 448)).to(torch.float8_e4m3fn).view(torch.uint8)
    dev = cuda_device
    D = torch.full((m, n), 9.0, dtype=torch.float32, device=dev)
    R.async_gemm(A.to(dev), B.to(dev), D, m, n, k, project=project)
    torch.cuda.synchronize()
    ref64, mag = oracle.gemm_fp8_f64(A.numpy(), B.numpy(), 1.0, 1.0)
    tol = 4 * np.sqrt(k) * 2.0 ** -24 * mag + 1e-30
    assert (np.abs(D.cpu().numpy().astype(np.float64) - ref64) <= tol).all()
    ref32 = oracle.gemm_fp8_f32(A.numpy(), B.numpy())
    mx, tot = oracle.deltas(D.cpu().numpy(), ref32)             # the reference's printed metric
    assert mx <= float(tol.max())


def test_reference_shape_rule(cuda_device):
    import rocm_dev_b200 as R
    dev = cuda_device
    z = torch.zeros(16, dtype=torch.uint8, device=dev)
    with pytest.raises(R.AsyncGemmShapeError):
        R.async_gemm(z, z, torch.zeros(1, device=dev), 17, 16, 64)
    with pytest.raises(R.AsyncGemmShapeError):
        R.async_gemm(z, z, torch.zeros(1, device=dev), 16, 40, 64, project="async_gemm_blanes")


def test_error_codes(cuda_device):
    import rocm_dev_b200 as R
    dev = cuda_device
    A = torch.zeros((16, 64), dtype=torch.uint8, device=dev)
    D = torch.zeros((16, 16), dtype=torch.bfloat16, device=dev)
    one = torch.ones(1, device=dev)
    L = R.lib()
    assert L.rdb_dense_gemm_fp8(A.data_ptr(), A.data_ptr(), one.data_ptr(), one.data_ptr(), D.data_ptr(), 16, 16, 60, 0) == 3
    assert L.rdb_dense_gemm_fp8(A.data_ptr(), A.data_ptr(), one.data_ptr(), one.data_ptr(), D.data_ptr(), 0, 16, 64, 0) == 8
    assert L.rdb_dense_gemm_fp8(A.data_ptr() + 4, A.data_ptr(), one.data_ptr(), one.data_ptr(), D.data_ptr(), 16, 16, 64, 0) == 7
    assert L.rdb_dense_gemm_fp8(A.data_ptr(), A.data_ptr(), None, one.data_ptr(), D.data_ptr(), 16, 16, 64, 0) == 6
