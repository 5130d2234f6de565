"""2:4 structured-sparse FP8 GEMM: the packer against the oracle's compressor
(CPU) and the kernel against the oracle's dense GEMM on the pruned matrix (GPU,
same tolerance as the dense paths)."""
import numpy as np
import pytest
import torch

from helpers import bf16_bits, check_gemm_parity


def _sparse_weights(N, K, seed):
    import rocm_dev_b200 as R
    from rocm_dev_b200 import quant
    g = torch.Generator().manual_seed(seed)
    W = (torch.randn((N, K), generator=g) * 0.02).bfloat16()
    Wq, sb = quant.quantize_per_tensor(R.prune_2of4(W))
    return Wq, sb


def test_prune_matches_oracle(oracle):
    import rocm_dev_b200 as R
    g = torch.Generator().manual_seed(0)
    W = torch.randn((32, 256), generator=g)
    W[0, :4] = torch.tensor([0.5, -0.5, 0.5, 0.1])
    W[1, :8] = 0
    assert np.array_equal(R.prune_2of4(W).numpy(), oracle.prune_2of4(W.numpy()))


def test_packer_matches_oracle_compressor(oracle):
    import rocm_dev_b200 as R
    N, K = 256, 512
    Wq, _ = _sparse_weights(N, K, 1)
    Wq[3, :4] = 0                      # empty group
    Wq[4, :4] = torch.tensor([0, 0, 0, 0x38], dtype=torch.uint8)
    Wq[5, :4] = torch.tensor([0x80, 0x40, 0, 0], dtype=torch.uint8)    # -0 is a zero
    vals, meta = R.pack_2of4(Wq)
    ovals, ometa, bad = oracle.compress_2of4(Wq.numpy())
    assert bad == 0 and np.array_equal(vals.numpy(), ovals)
    # unpack the tiled nibbles back to one byte per group and compare
    m = meta.numpy().reshape(N // 128, K // 128, 128, 16)
    lo, hi = m & 0xF, m >> 4
    per_group = np.stack([lo, hi], axis=-1).reshape(N // 128, K // 128, 128, 32)       # [tile][atom][row][chunk]
    per_group = per_group.transpose(0, 2, 1, 3).reshape(N, K // 4)
    assert np.array_equal(per_group, ometa)
    back = oracle.expand_2of4(vals.numpy(), per_group)
    nz = (Wq.numpy() & 0x7F) != 0
    assert np.array_equal(back[nz], Wq.numpy()[nz]) and not (back[~nz] & 0x7F).any()   # a padded slot may keep a -0 byte
    dense = Wq.clone()
    dense[0, :4] = 0x38
    with pytest.raises(R.RdbError):
        R.pack_2of4(dense)


def _check(oracle, dev, M, N, K, seed=0, split_k=0):
    import rocm_dev_b200 as R
    from rocm_dev_b200 import quant
    Wq, sb = _sparse_weights(N, K, seed)
    g = torch.Generator().manual_seed(seed + 1)
    Aq, sa = quant.quantize_per_tensor(torch.randn((M, K), generator=g).bfloat16())
    vals, meta = R.pack_2of4(Wq)
    out = R.sparse_gemm_fp8(Aq.to(dev), vals.to(dev), meta.to(dev), sa.to(dev), sb.to(dev), split_k=split_k)
    torch.cuda.synchronize()
    assert R.lib().rdb_device_status() == 0
    ref = oracle.gemm_fp8_bf16(Aq.numpy(), Wq.numpy(), sa.item(), sb.item())
    ref64, mag = oracle.gemm_fp8_f64(Aq.numpy(), Wq.numpy(), sa.item(), sb.item())
    return check_gemm_parity(bf16_bits(out), ref, ref64, mag, K)


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(16, 128, 256), (16, 128, 1024), (8, 256, 512), (64, 384, 2048), (256, 256, 1024),
                                   (100, 200, 768), (1, 2, 256)])
def test_small_shapes(cuda_device, oracle, M, N, K):
    _check(oracle, cuda_device, M, N, K, seed=M + N)


@pytest.mark.gpu
@pytest.mark.parametrize("split_k", [1, 2, 4])
def test_every_k_split(cuda_device, oracle, split_k):
    _check(oracle, cuda_device, 16, 512, 4096, seed=9, split_k=split_k)


@pytest.mark.gpu
@pytest.mark.parametrize("M", [16, 64, 256])
def test_config3_matches_oracle_and_own_dense_kernel(cuda_device, oracle, M):
    """N = K = 8192 (BASELINE config 3): oracle on the pruned matrix, and the
    library's dense kernel on the same pruned matrix (bit-identical fp32 sums
    are not required of two different tilings, so within 2 bf16 ulp)."""
    import rocm_dev_b200 as R
    from rocm_dev_b200 import quant
    from helpers import bf16_ulp_distance
    N = K = 8192
    r = _check(oracle, cuda_device, M, N, K, seed=M)
    assert r["rel_fro"] < 1e-2
    Wq, sb = _sparse_weights(N, K, M)
    Aq, sa = quant.quantize_per_tensor(torch.randn((M, K), generator=torch.Generator().manual_seed(M + 1)).bfloat16())
    dev = cuda_device
    vals, meta = R.pack_2of4(Wq)
    sp = R.sparse_gemm_fp8(Aq.to(dev), vals.to(dev), meta.to(dev), sa.to(dev), sb.to(dev))
    de = R.dense_gemm_fp8(Aq.to(dev), Wq.to(dev), sa.to(dev), sb.to(dev))
    assert bf16_ulp_distance(bf16_bits(sp), bf16_bits(de)).max() <= 2


@pytest.mark.gpu
def test_error_codes(cuda_device):
    import rocm_dev_b200 as R
    L = R.lib()
    dev = cuda_device
    z = torch.zeros(1 << 16, dtype=torch.uint8, device=dev)
    one = torch.ones(1, device=dev)
    D = torch.zeros(1 << 16, dtype=torch.bfloat16, device=dev)
    args = lambda M, N, K: (z.data_ptr(), z.data_ptr(), z.data_ptr(), one.data_ptr(), one.data_ptr(), D.data_ptr(), M, N, K, 0)  # noqa: E731
    assert L.rdb_sparse_gemm_fp8(*args(16, 128, 200)) == 3
    assert L.rdb_sparse_gemm_fp8(*args(257, 128, 256)) == 1
    assert L.rdb_sparse_gemm_fp8(*args(16, 127, 256)) == 2
    assert L.rdb_sparse_gemm_fp8(*args(0, 128, 256)) == 8
    assert L.rdb_sparse_meta_bytes(128, 100) == 0
