"""Comparison rules shared by the parity tests."""
from __future__ import annotations

import numpy as np


def bf16_bits(t) -> np.ndarray:
    """torch bf16 tensor -> uint16 bit patterns."""
    import torch
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def bf16_ulp_distance(a_bits: np.ndarray, b_bits: np.ndarray) -> np.ndarray:
    """Distance in units in the last place between bf16 bit patterns."""
    def ordered(b):
        b = b.astype(np.int32)
        return np.where(b & 0x8000, 0x8000 - (b & 0x7FFF), 0x8000 + b)
    return np.abs(ordered(a_bits) - ordered(b_bits))


def bf16_ulp_of(x: np.ndarray) -> np.ndarray:
    """Size of one bf16 ulp at magnitude |x| (float64)."""
    ax = np.maximum(np.abs(x), 2.0 ** -126)
    return 2.0 ** (np.floor(np.log2(ax)) - 7)


def check_gemm_parity(got_bits, ref_bits, ref64, mag, K, rel_fro=1e-2, ulps=2):
    """The stated tolerance: relative Frobenius error <= 1e-2 against the
    sequential-fp32 oracle, and every element within 2 bf16 ulp of it.  An
    element that misses the 2-ulp rule is adjudicated against the fp64 result:
    it still passes if its error is within 2 bf16 ulp of the fp64 value plus
    the fp32 summation-order noise 4*sqrt(K)*2^-24*sum|a*b|*scale (cancelling
    sums make the oracle itself that uncertain).  Returns a report dict."""
    got = bf16_to_f32(got_bits).astype(np.float64)
    ref = bf16_to_f32(ref_bits).astype(np.float64)
    fro = np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-30)
    dist = bf16_ulp_distance(got_bits, ref_bits)
    miss = dist > ulps
    tol64 = ulps * bf16_ulp_of(ref64) + 4.0 * np.sqrt(K) * 2.0 ** -24 * mag
    bad = miss & (np.abs(got - ref64) > tol64)
    report = {
        "rel_fro": float(fro),
        "max_ulp": int(dist.max()) if dist.size else 0,
        "beyond_2ulp_of_fp32_oracle": int(miss.sum()),
        "failing": int(bad.sum()),
        "bit_exact_fraction": float((dist == 0).mean()) if dist.size else 1.0,
    }
    assert np.isfinite(got).all(), "non-finite output"
    assert fro <= rel_fro, report
    assert report["failing"] == 0, report
    return report
