"""Host side of the skinny FP8 GEMM, mirroring the reference launchers.

Reference interface (paths within the reference project):
  - ``skinny_gemm_fastpath(A, B, D, scale_tensor, m, n, k)`` -
    projects/skinny_gemm/skinny_gemm_caller.cu:343-405
  - ``skinny_gemm(A, B, D, scale_tensor, m, n, k, b_stride, split_k, ...)`` -
    projects/skinny_gemm/skinny_gemm_caller.cu:20-340
  - ``HFRK_skinny_gemm(world_size).skinny_gemm_torch_binding(...)`` -
    projects/skinny_gemm/skinny_gemm_binding.cu:64-100
Differences, all forced by the target: bytes are OCP e4m3fn (the reference's
are AMD e4m3 FNUZ), D is bf16 (reference: fp16) and is overwritten rather than
accumulated into, and a second per-tensor scale exists (``scale_b``; the
reference-named wrappers pass 1).
"""
from __future__ import annotations

import ctypes as C
import enum

import torch

from ._lib import check, lib


class SkinnyGemmReturnCode(enum.IntEnum):
    """projects/skinny_gemm/skinny_gemm_caller.cu:9-17, extended."""
    SUCCESS = 0
    M_ABOVE_WARPTILE_M = 1
    N_NOT_EVEN = 2
    K_NOT_DIVISIBLE_BY_WARPTILE_K = 3
    TOO_MANY_WARPS = 4
    QSIZE_TOO_SMALL = 5
    INVALID_CONFIG = 6
    BAD_ALIGNMENT = 7
    BAD_SHAPE = 8
    CUDA_ERROR = 9
    DEVICE_TIMEOUT = 10
    SIZE_ABOVE_LIMIT = 11
    IO_ERROR = 12
    BAD_FILE = 13


_ones: dict[int, torch.Tensor] = {}


def _one(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _ones:
        _ones[idx] = torch.ones(1, dtype=torch.float32, device=device)
    return _ones[idx]


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _u8(t: torch.Tensor) -> torch.Tensor:
    return t if t.dtype == torch.uint8 else t.view(torch.uint8)


def skinny_gemm_fp8(A: torch.Tensor, B: torch.Tensor, scale_a: torch.Tensor, scale_b: torch.Tensor,
                    out: torch.Tensor | None = None) -> torch.Tensor:
    """D[M,N] = bf16((A . B^T) * scale_a * scale_b) on the current stream.

    A: [M,K] e4m3fn bytes (uint8 or float8_e4m3fn), M <= 32, contiguous.
    B: [N,K] e4m3fn bytes, K-contiguous (any row pitch that is a multiple of 16).
    scale_a, scale_b: one fp32 each, on the device.
    """
    assert A.is_cuda and B.is_cuda, "device tensors required (there is no CPU path)"
    A = _u8(A)
    B = _u8(B)
    M, K = A.shape
    N = B.shape[0]
    assert B.shape[1] == K and B.stride(1) == 1 and A.is_contiguous()
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=A.device)
    assert out.dtype == torch.bfloat16 and out.is_contiguous() and out.shape == (M, N)
    with torch.cuda.device(A.device):
        code = lib().rdb_skinny_gemm_fp8(A.data_ptr(), B.data_ptr(), scale_a.data_ptr(), scale_b.data_ptr(),
                                         out.data_ptr(), M, N, K, B.stride(0), _stream_ptr(A.device))
    check(code, "rdb_skinny_gemm_fp8")
    return out


OVERLAP_PRIOR_KERNEL = 1


def skinny_gemm_fp8_tuned(A, B, scale_a, scale_b, out, rows_per_tile=0, split_k=0, stages=0, flags=0) -> int:
    """Tuner entry (rdb_skinny_gemm_fp8_tuned): explicit tile height, K split,
    stage count and launch flags; returns the status code."""
    A = _u8(A)
    B = _u8(B)
    M, K = A.shape
    N = B.shape[0]
    with torch.cuda.device(A.device):
        return int(lib().rdb_skinny_gemm_fp8_tuned(A.data_ptr(), B.data_ptr(), scale_a.data_ptr(), scale_b.data_ptr(),
                                                   out.data_ptr(), M, N, K, B.stride(0), rows_per_tile, split_k,
                                                   stages, flags, _stream_ptr(A.device)))


GROUP_MAX = 32


class SkinnyProblem(C.Structure):
    """``rdb_skinny_problem`` of include/rocm_dev_b200.h."""
    _fields_ = [("A", C.c_void_p), ("B", C.c_void_p), ("scale_a", C.c_void_p), ("scale_b", C.c_void_p),
                ("D", C.c_void_p), ("M", C.c_int), ("N", C.c_int), ("K", C.c_int), ("ldb", C.c_int)]


def _problem_array(problems):
    arr = (SkinnyProblem * len(problems))()
    for i, (A, B, sa, sb, D) in enumerate(problems):
        A, B = _u8(A), _u8(B)
        M, K = A.shape
        arr[i] = SkinnyProblem(A.data_ptr(), B.data_ptr(), sa.data_ptr(), sb.data_ptr(), D.data_ptr(), M, B.shape[0], K,
                               B.stride(0))
    return arr


def skinny_gemm_fp8_grouped(problems, flags: int = 0) -> int:
    """A list of independent skinny GEMMs in one persistent launch
    (rdb_skinny_gemm_fp8_grouped) - the shape of the reference's timed region,
    BATCH back-to-back ``skinny_gemm_fastpath`` calls on different weights
    (projects/skinny_gemm/bench.cu:51-60).  ``problems``: up to 32 tuples
    ``(A, B, scale_a, scale_b, D)`` of device tensors with the meaning of
    ``skinny_gemm_fp8``.  ``flags``: 0 or ``OVERLAP_PRIOR_KERNEL`` (the launch may
    start streaming weights while the preceding kernel of the stream drains).
    Returns the status code."""
    dev = problems[0][0].device
    arr = _problem_array(problems)
    with torch.cuda.device(dev):
        return int(lib().rdb_skinny_gemm_fp8_grouped(arr, len(problems), flags, _stream_ptr(dev)))


def skinny_gemm_grouped_plan(shapes, ctas: int = 148):
    """Work split of a grouped call for ``shapes`` = [(M, N, K), ...]: (rows
    per unit of each problem, first unit of each CTA's range).  No GPU needed."""
    arr = (SkinnyProblem * len(shapes))()
    for i, (M, N, K) in enumerate(shapes):
        arr[i] = SkinnyProblem(None, None, None, None, None, M, N, K, K)
    rows = (C.c_int * len(shapes))()
    ranges = (C.c_int * (ctas + 1))()
    check(lib().rdb_skinny_gemm_grouped_plan(arr, len(shapes), ctas, rows, ranges), "rdb_skinny_gemm_grouped_plan")
    return list(rows), list(ranges)


def skinny_gemm_fastpath(A, B, D, scale_tensor, m: int, n: int, k: int) -> int:
    """Reference-named launcher: returns the status code instead of raising.

    Tensors may be torch CUDA tensors or raw device addresses (ints).
    """
    ptr = lambda t: t if isinstance(t, int) else t.data_ptr()  # noqa: E731
    dev = next((t.device for t in (A, B, D) if isinstance(t, torch.Tensor)), torch.device("cuda"))
    with torch.cuda.device(dev):
        return int(lib().rdb_skinny_gemm_fp8(ptr(A), ptr(B), ptr(scale_tensor), _one(torch.device(dev)).data_ptr(),
                                             ptr(D), m, n, k, k, 0))


def skinny_gemm(A, B, D, scale_tensor, m, n, k, b_stride, split_k, A_producers, B_producers, consumers,
                b_lanes, qsize, op_m, ops, stream=None) -> int:
    """Reference-named full launcher; tuning ints are validated like the
    reference does and used as hints (split_k, qsize) or ignored."""
    ptr = lambda t: t if isinstance(t, int) else t.data_ptr()  # noqa: E731
    dev = next((t.device for t in (A, B, D) if isinstance(t, torch.Tensor)), torch.device("cuda"))
    with torch.cuda.device(dev):
        s = _stream_ptr(dev) if stream is None else (stream if isinstance(stream, int) else stream.cuda_stream)
        return int(lib().rdb_skinny_gemm_fp8_hinted(
            ptr(A), ptr(B), ptr(scale_tensor), _one(torch.device(dev)).data_ptr(), ptr(D), m, n, k, b_stride,
            split_k, A_producers, B_producers, consumers, b_lanes, qsize, op_m, ops, s))


class HFRK_skinny_gemm:
    """Mirror of the pybind class of projects/skinny_gemm/skinny_gemm_binding.cu."""

    def __init__(self, world_size: int):
        self.world_size = int(world_size)

    def skinny_gemm_torch_binding(self, A, B, D, scale_tensor, split_k, A_producers, B_producers, consumers,
                                  b_lanes, qsize, ops) -> int:
        # B arrives as a [K,N] view of [N,K] K-contiguous storage; stride(1) is
        # the row pitch (skinny_gemm_binding.cu:36-39).
        m, k = A.size(0), A.size(1)
        n = B.size(1)
        b_stride = B.stride(1)
        op_m = 8 if m <= 8 else (16 if m <= 16 else 32)
        return skinny_gemm(_u8(A), _u8(B), D, scale_tensor, m, n, k, b_stride, split_k, A_producers, B_producers,
                           consumers, b_lanes, qsize, op_m, ops)


def skinny_gemm_fp8_host(A: torch.Tensor, B: torch.Tensor, scale_a: torch.Tensor, scale_b: torch.Tensor,
                         out: torch.Tensor, device="cuda") -> torch.Tensor:
    """Same contraction with HOST (ideally pinned) tensors through
    ``rdb_skinny_gemm_fp8_host``: the library copies every input to the device,
    runs the kernel and copies the bf16 result back into ``out``; everything is
    queued on the current stream and the call returns after the result has
    arrived."""
    dev = torch.device(device)
    A, B = _u8(A), _u8(B)
    assert not A.is_cuda and not B.is_cuda and not out.is_cuda, "host tensors expected"
    assert A.is_contiguous() and B.stride(1) == 1 and out.is_contiguous() and out.dtype == torch.bfloat16
    M, K = A.shape
    N = B.shape[0]
    with torch.cuda.device(dev):
        code = lib().rdb_skinny_gemm_fp8_host(A.data_ptr(), B.data_ptr(), scale_a.data_ptr(), scale_b.data_ptr(),
                                              out.data_ptr(), M, N, K, B.stride(0), _stream_ptr(dev))
    check(code, "rdb_skinny_gemm_fp8_host")
    return out
