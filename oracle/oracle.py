"""ctypes front-end of the CPU oracle (oracle.c).

TEST INFRASTRUCTURE ONLY.  Importers are limited to the test-suite, the smoke
check and the CPU-baseline leg of the benchmark; the product package never
imports this module.  Parity status: unpinned against reference outputs (the
reference has no golden vectors and its host code needs the ROCm toolchain);
pinned against the known-answer vectors under tests/golden/.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liboracle.so")


def build(force: bool = False) -> str:
    """Compile oracle.c with gcc if the shared object is missing or stale."""
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "liboracle.so"], stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        _lib.orc_e4m3fn_decode.restype = C.c_float
        _lib.orc_e4m3fn_decode.argtypes = [C.c_uint8]
        _lib.orc_e4m3fn_encode.restype = C.c_uint8
        _lib.orc_e4m3fn_encode.argtypes = [C.c_float]
        _lib.orc_bf16_encode.restype = C.c_uint16
        _lib.orc_bf16_encode.argtypes = [C.c_float]
        _lib.orc_compress_2of4.restype = C.c_int
        _lib.orc_num_threads.restype = C.c_int
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


def num_threads() -> int:
    return int(lib().orc_num_threads())


# ------------------------------------------------------------------ codecs
def e4m3fn_decode(q) -> np.ndarray:
    q = _c(q, np.uint8)
    out = np.empty(q.shape, np.float32)
    lib().orc_e4m3fn_decode_n(_p(q), _p(out), C.c_size_t(q.size))
    return out


def e4m3fn_encode(x) -> np.ndarray:
    x = _c(x, np.float32)
    out = np.empty(x.shape, np.uint8)
    lib().orc_e4m3fn_encode_n(_p(x), _p(out), C.c_size_t(x.size))
    return out


def bf16_encode(x) -> np.ndarray:
    """fp32 -> bf16 bit patterns (uint16), round-to-nearest-even."""
    x = _c(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().orc_bf16_encode_n(_p(x), _p(out), C.c_size_t(x.size))
    return out


def bf16_decode(h) -> np.ndarray:
    h = _c(h, np.uint16)
    return (h.astype(np.uint32) << 16).view(np.float32)


# -------------------------------------------------------------- quantisers
def quantize_per_tensor(x):
    """Returns (q uint8 of x.shape, scale float32): scale = amax/448."""
    x = _c(x, np.float32)
    q = np.empty(x.shape, np.uint8)
    s = C.c_float()
    lib().orc_quantize_per_tensor(_p(x), C.c_size_t(x.size), _p(q), C.byref(s))
    return q, np.float32(s.value)


def quantize_blocks128(x_bf16):
    """x_bf16: uint16 bit patterns, size % 128 == 0 -> (q uint8, scales f32)."""
    x = _c(x_bf16, np.uint16)
    assert x.size % 128 == 0
    q = np.empty(x.shape, np.uint8)
    s = np.empty(x.size // 128, np.float32)
    lib().orc_quantize_blocks128(_p(x), C.c_size_t(x.size), _p(q), _p(s))
    return q, s


# -------------------------------------------------------------------- GEMMs
def gemm_fp8_bf16(A, B, scale_a, scale_b, ldb=None) -> np.ndarray:
    """bf16 bit patterns [M,N] of (A*sa)(B*sb)^T, sequential fp32 accumulate."""
    A = _c(A, np.uint8)
    B = _c(B, np.uint8)
    M, K = A.shape
    N = B.shape[0]
    ldb = B.shape[1] if ldb is None else ldb
    D = np.empty((M, N), np.uint16)
    lib().orc_gemm_fp8_bf16(_p(A), _p(B), C.c_float(scale_a), C.c_float(scale_b), _p(D),
                            C.c_int(M), C.c_int(N), C.c_int(K), C.c_int(ldb))
    return D


def gemm_fp8_f64(A, B, scale_a, scale_b, ldb=None):
    """(D float64 [M,N], mag float64 [M,N]): fp64-accumulated result and
    sum_k |a*b|*scale, the magnitude summation-order noise scales with."""
    A = _c(A, np.uint8)
    B = _c(B, np.uint8)
    M, K = A.shape
    N = B.shape[0]
    ldb = B.shape[1] if ldb is None else ldb
    D = np.empty((M, N), np.float64)
    mag = np.empty((M, N), np.float64)
    lib().orc_gemm_fp8_f64(_p(A), _p(B), C.c_float(scale_a), C.c_float(scale_b), _p(D), _p(mag),
                           C.c_int(M), C.c_int(N), C.c_int(K), C.c_int(ldb))
    return D, mag


def gemm_fp8_f32(A, B) -> np.ndarray:
    A = _c(A, np.uint8)
    B = _c(B, np.uint8)
    M, K = A.shape
    N = B.shape[0]
    D = np.empty((M, N), np.float32)
    lib().orc_gemm_fp8_f32(_p(A), _p(B), _p(D), C.c_int(M), C.c_int(N), C.c_int(K))
    return D


# ------------------------------------------------------------------ reduce
def tiled_sum_reduce(A, B) -> np.ndarray:
    A = _c(A, np.float32)
    B = _c(B, np.float32)
    b, m, n = A.shape
    D = np.empty((m, n), np.float32)
    lib().orc_tiled_sum_reduce(_p(A), _p(B), _p(D), C.c_int(b), C.c_int(m), C.c_int(n))
    return D


def allreduce_fp8(xs_bf16):
    """xs_bf16: uint16 [nranks, n] -> (out bf16 bits [n], q uint8 [nranks,n],
    scales f32 [nranks, n/128])."""
    xs = _c(xs_bf16, np.uint16)
    r, n = xs.shape
    assert n % 128 == 0
    out = np.empty(n, np.uint16)
    q = np.empty((r, n), np.uint8)
    s = np.empty((r, n // 128), np.float32)
    lib().orc_allreduce_fp8(_p(xs), C.c_int(r), C.c_size_t(n), _p(out), _p(q), _p(s))
    return out, q, s


def allreduce_fp8_regather(xs_bf16):
    """Second variant of the allreduce (FP8 all-gather): the bf16 result of
    `allreduce_fp8` is block-quantised once more and decoded,
    out = bf16(fp32(code) * scale).  No reference counterpart (the allreduce is
    specified by configuration text only); defined here as the composition of
    the two primitives above."""
    y, _, _ = allreduce_fp8(xs_bf16)
    q, s = quantize_blocks128(y)
    dec = e4m3fn_decode(np.arange(256, dtype=np.uint8))
    prod = dec[q].astype(np.float32) * np.repeat(s.astype(np.float32), 128)
    return bf16_encode(prod.astype(np.float32))


# --------------------------------------------------------------- 2:4 sparse
def prune_2of4(W) -> np.ndarray:
    W = np.array(W, dtype=np.float32, order="C", copy=True)
    N, K = W.shape
    assert K % 4 == 0
    lib().orc_prune_2of4(_p(W), C.c_int(N), C.c_int(K))
    return W


def compress_2of4(Wq):
    """Wq uint8 [N,K] (2:4) -> (vals [N,K/2], meta [N,K/4], bad_groups)."""
    Wq = _c(Wq, np.uint8)
    N, K = Wq.shape
    vals = np.empty((N, K // 2), np.uint8)
    meta = np.empty((N, K // 4), np.uint8)
    bad = lib().orc_compress_2of4(_p(Wq), C.c_int(N), C.c_int(K), _p(vals), _p(meta))
    return vals, meta, int(bad)


def expand_2of4(vals, meta) -> np.ndarray:
    vals = _c(vals, np.uint8)
    meta = _c(meta, np.uint8)
    N, K4 = meta.shape
    Wq = np.empty((N, K4 * 4), np.uint8)
    lib().orc_expand_2of4(_p(vals), _p(meta), C.c_int(N), C.c_int(K4 * 4), _p(Wq))
    return Wq


def deltas(x, ref):
    """(max_delta, total_delta) as the reference drivers print them."""
    x = _c(x, np.float32).ravel()
    ref = _c(ref, np.float32).ravel()
    mx, tot = C.c_float(), C.c_float()
    lib().orc_deltas(_p(x), _p(ref), C.c_size_t(x.size), C.byref(mx), C.byref(tot))
    return mx.value, tot.value
