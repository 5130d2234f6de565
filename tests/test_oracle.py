"""CPU tests: the oracle against the committed known-answer vectors."""
import json
import os

import numpy as np
import pytest
import torch

GOLD = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def ka():
    with open(os.path.join(GOLD, "known_answers.json")) as f:
        return json.load(f)


def test_decode_all_256_codes(oracle, ka):
    got = oracle.e4m3fn_decode(np.arange(256, dtype=np.uint8)).view(np.uint32)
    want = np.array(ka["e4m3fn_decode_bits"], np.uint32)
    nan = np.isnan(want.view(np.float32))
    assert np.array_equal(got[~nan], want[~nan])
    assert np.isnan(got.view(np.float32)[nan]).all() and nan.sum() == 2
    # format facts
    f = got.view(np.float32)
    assert f[0x38] == 1.0 and f[0x7E] == 448.0 and f[0x77] == 240.0 and f[0x01] == 2.0 ** -9
    assert np.signbit(f[0x80]) and f[0x80] == 0.0


def test_encode_every_bf16_pattern(oracle):
    want = np.load(os.path.join(GOLD, "e4m3fn_encode_of_bf16.npy"))
    bits = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    got = oracle.e4m3fn_encode(oracle.bf16_decode(bits))
    assert np.array_equal(got, want)


def test_encode_cases(oracle, ka):
    x = np.array(ka["encode_cases"]["x_bits"], np.uint32).view(np.float32)
    assert oracle.e4m3fn_encode(x).tolist() == ka["encode_cases"]["code"]


def test_encode_decode_round_trip(oracle):
    codes = np.array([c for c in range(256) if (c & 0x7F) != 0x7F], np.uint8)
    assert np.array_equal(oracle.e4m3fn_encode(oracle.e4m3fn_decode(codes)), codes)


def test_bf16_rounding(oracle, ka):
    x = np.array(ka["bf16_cases"]["x_bits"], np.uint32).view(np.float32)
    assert oracle.bf16_encode(x).tolist() == ka["bf16_cases"]["bf16"]


def test_tiny_gemm_known_answer(oracle, ka):
    t = ka["tiny_gemm"]
    D = oracle.gemm_fp8_bf16(np.array(t["A"], np.uint8), np.array(t["B"], np.uint8), t["scale_a"], t["scale_b"])
    assert D.tolist() == t["D_bf16"]
    D64, mag = oracle.gemm_fp8_f64(np.array(t["A"], np.uint8), np.array(t["B"], np.uint8), t["scale_a"], t["scale_b"])
    assert np.array_equal(oracle.bf16_encode(D64.astype(np.float32)), D)
    assert (mag >= np.abs(D64) - 1e-12).all()


def test_blocks128_known_answer(oracle, ka):
    b = ka["blocks128"]
    q, s = oracle.quantize_blocks128(np.array(b["x_bf16"], np.uint16))
    assert q.tolist() == b["q"]
    assert s.view(np.uint32).tolist() == b["scale_bits"]


def test_quantizers_match_host_library(oracle):
    """The product's host quantisers (torch) and the oracle agree bit for bit."""
    from rocm_dev_b200 import quant
    g = torch.Generator().manual_seed(3)
    x = torch.randn(64, 512, generator=g) * 0.02
    q, s = quant.quantize_per_tensor(x)
    oq, os_ = oracle.quantize_per_tensor(x.numpy())
    assert np.array_equal(q.numpy(), oq) and np.float32(s.item()) == os_
    xb = torch.randn(8, 1024, generator=g).bfloat16()
    q2, s2 = quant.quantize_blocks128(xb)
    oq2, os2 = oracle.quantize_blocks128(xb.view(torch.int16).numpy().view(np.uint16).ravel())
    assert np.array_equal(q2.numpy().ravel(), oq2) and np.array_equal(s2.numpy(), os2)
    z, sz = quant.quantize_per_tensor(torch.zeros(16))
    assert sz.item() == 1.0 and not z.any()


def test_gemm_oracle_against_torch_fp64(oracle):
    from rocm_dev_b200 import quant
    Aq, Bq, sa, sb = quant.synthetic_gemm_operands(5, 96, 256, seed=1)
    D64, _ = oracle.gemm_fp8_f64(Aq.numpy(), Bq.numpy(), sa.item(), sb.item())
    ref = (Aq.view(torch.float8_e4m3fn).double() @ Bq.view(torch.float8_e4m3fn).double().T) * float(
        np.float32(sa.item()) * np.float32(sb.item()))
    assert np.allclose(D64, ref.numpy(), rtol=1e-12, atol=0)
    D = oracle.gemm_fp8_bf16(Aq.numpy(), Bq.numpy(), sa.item(), sb.item())
    from helpers import bf16_ulp_distance
    assert bf16_ulp_distance(D, oracle.bf16_encode(D64.astype(np.float32))).max() <= 1
    # row pitch larger than K reads the same values
    Bp = np.zeros((96, 320), np.uint8)
    Bp[:, :256] = Bq.numpy()
    Dp = oracle.gemm_fp8_bf16(Aq.numpy(), Bp, sa.item(), sb.item(), ldb=320)
    assert np.array_equal(Dp, D)


def test_gemm_f32_oracle_is_unscaled_sequential(oracle):
    rng = np.random.default_rng(0)
    A = rng.integers(0, 0x78, (4, 64), dtype=np.uint8)
    B = rng.integers(0, 0x78, (8, 64), dtype=np.uint8)
    D = oracle.gemm_fp8_f32(A, B)
    a, b = oracle.e4m3fn_decode(A), oracle.e4m3fn_decode(B)
    want = np.zeros((4, 8), np.float32)
    for i in range(4):
        for j in range(8):
            acc = np.float32(0)
            for l in range(64):
                acc = np.float32(acc + a[i, l] * b[j, l])
            want[i, j] = acc
    assert np.array_equal(D, want)


def test_tiled_sum_reduce_oracle(oracle):
    rng = np.random.default_rng(1)
    A = (rng.random((3, 8, 64), dtype=np.float32) - 0.5)
    B = (rng.random((3, 8, 64), dtype=np.float32) - 0.5)
    D = oracle.tiled_sum_reduce(A, B)
    want = np.zeros((8, 64), np.float32)
    for b in range(3):
        want += A[b] + B[b]
    assert np.array_equal(D, want)
    assert np.array_equal(oracle.tiled_sum_reduce(A[:0], B[:0]), np.zeros((8, 64), np.float32))


def test_allreduce_oracle_properties(oracle):
    g = torch.Generator().manual_seed(5)
    xs = torch.randn(4, 2048, generator=g).bfloat16()
    bits = xs.view(torch.int16).numpy().view(np.uint16)
    out, q, s = oracle.allreduce_fp8(bits)
    # encodings equal the standalone quantiser
    for r in range(4):
        qr, sr = oracle.quantize_blocks128(bits[r])
        assert np.array_equal(q[r], qr) and np.array_equal(s[r], sr)
    # the result is the rank-ordered fp32 sum of the dequantised values
    deq = oracle.e4m3fn_decode(q) * np.repeat(s, 128, axis=1)
    acc = np.zeros(2048, np.float32)
    for r in range(4):
        acc = (acc + deq[r]).astype(np.float32)
    assert np.array_equal(out, oracle.bf16_encode(acc))
    # close to the unquantised sum
    exact = xs.float().sum(0).numpy()
    got = oracle.bf16_decode(out)
    assert np.linalg.norm(got - exact) / np.linalg.norm(exact) < 5e-2
    # one rank: the result is the bf16 rounding of the dequantised input
    out1, q1, s1 = oracle.allreduce_fp8(bits[:1])
    assert np.array_equal(out1, oracle.bf16_encode(oracle.e4m3fn_decode(q1[0]) * np.repeat(s1[0], 128)))


def test_prune_and_compress_2of4(oracle):
    g = torch.Generator().manual_seed(9)
    W = (torch.randn(16, 64, generator=g) * 0.02).numpy()
    W[0, :4] = [0.5, -0.5, 0.5, 0.1]          # tie -> lowest indices kept
    W[1, :4] = [0.0, 0.0, 0.0, 0.0]
    P = oracle.prune_2of4(W)
    assert ((P.reshape(-1, 4) != 0).sum(1) <= 2).all()
    assert P[0, :4].tolist() == [0.5, -0.5, 0.0, 0.0]
    kept = np.sort(np.abs(P.reshape(-1, 4)), 1)[:, 2:]
    want = np.sort(np.abs(W.reshape(-1, 4)), 1)[:, 2:]
    assert np.array_equal(kept, want)
    from rocm_dev_b200 import quant
    q, _ = quant.quantize_per_tensor(torch.from_numpy(P))
    vals, meta, bad = oracle.compress_2of4(q.numpy())
    assert bad == 0 and vals.shape == (16, 32) and meta.shape == (16, 16)
    assert ((meta & 3) < (meta >> 2)).all()
    back = oracle.expand_2of4(vals, meta)
    # -0 bytes (0x80) count as zero and are dropped by the compressor
    qz = q.numpy().copy()
    qz[(qz & 0x7F) == 0] = 0
    assert np.array_equal(back, qz)


def test_deltas_metric(oracle):
    mx, tot = oracle.deltas(np.array([1.0, 2.0, 4.0]), np.array([1.5, 2.0, 3.0]))
    assert mx == 1.0 and tot == 1.5
