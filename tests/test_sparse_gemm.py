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


def test_file_round_trip_and_rejections(tmp_path, oracle):
    """The on-disk form of packed 2:4 weights: what is written comes back bit for
    bit with its shape and scale; files that are not of the format, are damaged,
    or do not hold a 2:4 selection are refused with the documented codes."""
    import struct
    import rocm_dev_b200 as R
    N, K = 200, 512                                   # a last tile with fewer than 128 rows
    Wq, sb = _sparse_weights(N, K, 3)
    vals, meta = R.pack_2of4(Wq)
    path = tmp_path / "w.rdb24"
    R.save_2of4(path, vals, meta, sb.item())
    raw = path.read_bytes()
    assert raw[:6] == b"RDB24W" and struct.unpack_from("<II", raw, 8) == (1, 64)
    assert struct.unpack_from("<ii", raw, 16) == (N, K) and len(raw) == 64 + vals.numel() + meta.numel()
    v2, m2, s2 = R.load_2of4(path)
    assert torch.equal(v2, vals) and torch.equal(m2, meta)
    assert np.float32(s2).tobytes() == sb.numpy().tobytes()
    # expanding what was read gives back the pruned matrix (the oracle's expander is the checker)
    m = m2.numpy().reshape(-1, K // 128, 128, 16)
    per_group = np.stack([m & 0xF, m >> 4], axis=-1).reshape(-1, K // 128, 128, 32).transpose(0, 2, 1, 3).reshape(-1, K // 4)[:N]
    back = oracle.expand_2of4(v2.numpy(), per_group)
    nz = (Wq.numpy() & 0x7F) != 0
    assert np.array_equal(back[nz], Wq.numpy()[nz]) and not (back[~nz] & 0x7F).any()
    # straight from the uncompressed bytes, and the refusal of a matrix that is not 2:4
    L = R.lib()
    p2 = tmp_path / "direct.rdb24"
    assert L.rdb_sparse_file_pack_and_write(str(p2).encode(), Wq.data_ptr(), sb.item(), N, K) == 0
    assert p2.read_bytes() == raw
    dense = Wq.clone()
    dense[7, 8:12] = 0x38
    assert L.rdb_sparse_file_pack_and_write(str(tmp_path / "no.rdb24").encode(), dense.data_ptr(), 1.0, N, K) == 6

    def refused(mutated: bytes) -> int:
        q = tmp_path / "bad.rdb24"
        q.write_bytes(mutated)
        try:
            R.load_2of4(q)
        except R.RdbError as e:
            return e.code
        return 0

    assert refused(b"NOTRDB24" + raw[8:]) == 13                                   # magic
    assert refused(raw[:8] + struct.pack("<I", 2) + raw[12:]) == 13               # version
    assert refused(raw[:-100]) == 13                                              # truncated
    assert refused(raw + b"x") == 13                                              # trailing bytes
    flipped = bytearray(raw)
    flipped[64 + 1000] ^= 0x10
    assert refused(bytes(flipped)) == 13                                          # checksum
    assert refused(raw[:16] + struct.pack("<i", N + 1) + raw[20:]) == 13          # header disagrees with the sizes
    # an intact file (valid checksum) whose metadata is not an ascending pair per group: not a 2:4 selection
    bad_meta = bytearray(raw)
    bad_meta[64 + vals.numel()] = 0x00                                           # idx0 == idx1 == 0
    h = 1469598103934665603
    for b in bytes(bad_meta[64:]):
        h = ((h ^ b) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    bad_meta[48:56] = struct.pack("<Q", h)
    assert refused(bytes(bad_meta)) == 6
    assert L.rdb_sparse_file_write(str(tmp_path / "w2").encode(), vals.data_ptr(), bytes(bad_meta[64 + vals.numel():]), 1.0, N, K) == 6
    with pytest.raises(R.RdbError) as e:
        R.load_2of4(tmp_path / "missing.rdb24")
    assert e.value.code == 12


@pytest.mark.gpu
def test_weights_loaded_from_a_file_give_the_same_product(cuda_device, oracle, tmp_path):
    import rocm_dev_b200 as R
    from rocm_dev_b200 import quant
    M, N, K = 16, 512, 1024
    Wq, sb = _sparse_weights(N, K, 5)
    vals, meta = R.pack_2of4(Wq)
    R.save_2of4(tmp_path / "w.rdb24", vals, meta, sb.item())
    v2, m2, s2 = R.load_2of4(tmp_path / "w.rdb24")
    Aq, sa = quant.quantize_per_tensor(torch.randn((M, K), generator=torch.Generator().manual_seed(6)).bfloat16())
    dev = cuda_device
    a = R.sparse_gemm_fp8(Aq.to(dev), vals.to(dev), meta.to(dev), sa.to(dev), sb.to(dev))
    b = R.sparse_gemm_fp8(Aq.to(dev), v2.to(dev), m2.to(dev), sa.to(dev), torch.tensor([s2], device=dev))
    assert torch.equal(a, b)


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
                                   (100, 200, 768), (1, 2, 256), (16, 20480, 1024), (40, 19200, 512)])
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
    library's dense kernel on the same pruned matrix.  The two kernels cut K at
    different places, so their fp32 sums differ in the last bits: nearly every
    element within 2 bf16 ulp, the rest explained by summation order (both meet
    the oracle with the fp64 adjudication), relative Frobenius distance tiny."""
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
    dist = bf16_ulp_distance(bf16_bits(sp), bf16_bits(de))
    assert (dist <= 2).mean() > 0.999
    assert ((sp.float() - de.float()).norm() / de.float().norm()).item() < 1e-3


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K,split_k", [(16, 1024, 4096, 0), (64, 512, 2048, 2), (200, 384, 1024, 1)])
def test_launches_that_overlap_their_predecessor(cuda_device, oracle, M, N, K, split_k):
    """OVERLAP_PRIOR_KERNEL: a chain of launches in which each one's activations are the previous one's business
    (here: a kernel that rewrites A between the GEMMs) gives the bits of ordinary launches."""
    import rocm_dev_b200 as R
    from rocm_dev_b200 import quant
    dev = cuda_device
    Wq, sb = _sparse_weights(N, K, 3)
    vals, meta = R.pack_2of4(Wq)
    vals, meta, dsb = vals.to(dev), meta.to(dev), sb.to(dev)
    acts = [quant.quantize_per_tensor(torch.randn((M, K), generator=torch.Generator().manual_seed(40 + i)).bfloat16()) for i in range(3)]
    A = torch.empty((M, K), dtype=torch.uint8, device=dev)
    sa = torch.empty(1, dtype=torch.float32, device=dev)
    outs = {}
    for flags in (0, R.OVERLAP_PRIOR_KERNEL):
        res = []
        for Aq, s in acts:
            A.copy_(Aq.to(dev))                       # the preceding kernels of the stream write A and its scale
            sa.copy_(s.to(dev))
            res.append(R.sparse_gemm_fp8(A, vals, meta, sa, dsb, split_k=split_k, flags=flags).clone())
        torch.cuda.synchronize()
        assert R.lib().rdb_device_status() == 0
        outs[flags] = res
    for a, b in zip(outs[0], outs[R.OVERLAP_PRIOR_KERNEL]):
        assert torch.equal(a, b)
    ref = oracle.gemm_fp8_bf16(acts[2][0].numpy(), Wq.numpy(), acts[2][1].item(), sb.item())
    ref64, mag = oracle.gemm_fp8_f64(acts[2][0].numpy(), Wq.numpy(), acts[2][1].item(), sb.item())
    check_gemm_parity(bf16_bits(outs[R.OVERLAP_PRIOR_KERNEL][2]), ref, ref64, mag, K)
    with pytest.raises(Exception):
        R.sparse_gemm_fp8(A, vals, meta, sa, dsb, flags=2)


@pytest.mark.gpu
@pytest.mark.parametrize("M", [8, 64, 200])
def test_a_list_of_gemms_in_one_launch(cuda_device, oracle, M):
    """rdb_sparse_gemm_fp8_grouped: problems of different N and K that share the batch - each result equals the
    oracle's, and the bits of the single call with the same K split; with the overlap flag as well.  Lists whose
    batch sizes differ, empty lists and over-long lists are refused."""
    import rocm_dev_b200 as R
    from rocm_dev_b200 import quant
    dev = cuda_device
    shapes = [(384, 1024), (128, 2048), (1000, 1024), (256, 1024)]
    split = 4 if M <= 64 else 1          # 14 tiles in all: clusters of four for a narrow batch, none for a wide one
    probs, refs = [], []
    for i, (N, K) in enumerate(shapes):
        Wq, sb = _sparse_weights(N, K, 50 + i)
        vals, meta = R.pack_2of4(Wq)
        Aq, sa = quant.quantize_per_tensor(torch.randn((M, K), generator=torch.Generator().manual_seed(60 + i)).bfloat16())
        D = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
        probs.append((Aq.to(dev), vals.to(dev), meta.to(dev), sa.to(dev), sb.to(dev), D))
        refs.append((Aq, Wq, sa, sb, K))
    for flags in (0, R.OVERLAP_PRIOR_KERNEL):
        for p in probs:
            p[5].zero_()
        assert R.sparse_gemm_fp8_grouped(probs, flags=flags) == 0
        torch.cuda.synchronize()
        assert R.lib().rdb_device_status() == 0
        for (A, vals, meta, sa, sb, D), (Aq, Wq, hsa, hsb, K) in zip(probs, refs):
            ref = oracle.gemm_fp8_bf16(Aq.numpy(), Wq.numpy(), hsa.item(), hsb.item())
            ref64, mag = oracle.gemm_fp8_f64(Aq.numpy(), Wq.numpy(), hsa.item(), hsb.item())
            check_gemm_parity(bf16_bits(D), ref, ref64, mag, K)
            single = R.sparse_gemm_fp8(A, vals, meta, sa, sb, split_k=split)
            assert torch.equal(D, single)
    other = list(probs[0])
    other[0] = torch.zeros((M + 1, shapes[0][1]), dtype=torch.uint8, device=dev)
    other[5] = torch.zeros((M + 1, shapes[0][0]), dtype=torch.bfloat16, device=dev)
    assert R.sparse_gemm_fp8_grouped([probs[1], tuple(other)]) == 6
    assert R.lib().rdb_sparse_gemm_fp8_grouped(None, 0, 0, None) == 6
    assert R.sparse_gemm_fp8_grouped(probs * 3) == 6


@pytest.mark.gpu
def test_step_trace(cuda_device):
    """rdb_sparse_gemm_trace: the first CTA's eight stamps of a launch are in order (the split-K slot only when the
    launch splits K) and switching it off stops the writes."""
    import rocm_dev_b200 as R
    from rocm_dev_b200 import quant
    dev = cuda_device
    M, N, K = 16, 512, 4096
    Wq, sb = _sparse_weights(N, K, 5)
    vals, meta = R.pack_2of4(Wq)
    Aq, sa = quant.quantize_per_tensor(torch.randn((M, K), generator=torch.Generator().manual_seed(6)).bfloat16())
    args = (Aq.to(dev), vals.to(dev), meta.to(dev), sa.to(dev), sb.to(dev))
    R.sparse_gemm_fp8(*args, split_k=2)
    torch.cuda.synchronize()
    tr = torch.zeros(2 * 8, dtype=torch.int64, device=dev)
    assert R.lib().rdb_sparse_gemm_trace(tr.data_ptr(), 2) == 0
    try:
        R.sparse_gemm_fp8(*args, split_k=2)
        R.sparse_gemm_fp8(*args, split_k=1)
        torch.cuda.synchronize()
    finally:
        assert R.lib().rdb_sparse_gemm_trace(None, 0) == 0
    t = tr.cpu().numpy().reshape(2, 8)
    assert (t[0] > 0).all() and (np.diff(t[0]) >= 0).all()
    assert t[1][5] == 0 and (np.diff(t[1][[0, 1, 2, 3, 4, 6, 7]]) >= 0).all() and t[1][0] >= t[0][7]
    tr.zero_()
    R.sparse_gemm_fp8(*args)
    torch.cuda.synchronize()
    assert int(tr.abs().sum().item()) == 0
    assert R.lib().rdb_sparse_gemm_trace(tr.data_ptr(), 0) == 6


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
