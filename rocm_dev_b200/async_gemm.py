"""Host side of the dense FP8 GEMM, mirroring the reference's async_gemm launchers.

Reference interface (paths within the reference project): the three projects
share ``template <class T> void async_gemm(const fp8* A, const fp8* B, T* D,
int m, int n, int k)`` -
projects/async_gemm_16x16x64/src.cu:54-82 (tile 16x16, k % 64),
projects/async_gemm_blanes/sparse_k.cu:46-80 (tile 16x48),
projects/async_gemm_sparse/sparse_k.cu:45-75 (tile 8x64).
They write unscaled fp32 and exit(1) when a shape does not divide their tile;
the mirror raises ``AsyncGemmShapeError`` in that case.  The new primary entry
``dense_gemm_fp8`` takes the two per-tensor scales and writes bf16.
"""
from __future__ import annotations

import torch

from ._lib import check, lib

# (WARPTILE_M, WARPTILE_N, WARPTILE_K) of each reference project
# (core.cu of the respective project).
PROJECT_TILES = {
    "async_gemm_16x16x64": (16, 16, 64),
    "async_gemm_blanes": (16, 48, 64),
    "async_gemm_sparse": (8, 64, 64),
}


class AsyncGemmShapeError(ValueError):
    """The reference prints a message and calls exit(1) for these shapes."""


def _u8(t: torch.Tensor) -> torch.Tensor:
    return t if t.dtype == torch.uint8 else t.view(torch.uint8)


def _stream(dev) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


def dense_gemm_fp8(A: torch.Tensor, B: torch.Tensor, scale_a: torch.Tensor, scale_b: torch.Tensor,
                   out: torch.Tensor | None = None, tile_rows: int = 0, max_ctas: int = 0) -> torch.Tensor:
    """D[M,N] = bf16((A . B^T) * scale_a * scale_b); A [M,K], B [N,K] e4m3fn bytes."""
    assert A.is_cuda and B.is_cuda and A.is_contiguous() and B.is_contiguous()
    A, B = _u8(A), _u8(B)
    M, K = A.shape
    N = B.shape[0]
    assert B.shape[1] == K
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=A.device)
    assert out.dtype == torch.bfloat16 and out.is_contiguous() and out.shape == (M, N)
    with torch.cuda.device(A.device):
        code = lib().rdb_dense_gemm_fp8_tuned(A.data_ptr(), B.data_ptr(), scale_a.data_ptr(), scale_b.data_ptr(),
                                              out.data_ptr(), M, N, K, tile_rows, max_ctas, _stream(A.device))
    check(code, "rdb_dense_gemm_fp8")
    return out


def async_gemm(A, B, D, m: int, n: int, k: int, project: str = "async_gemm_16x16x64") -> None:
    """Reference-named launcher: D [m,n] fp32 = A . B^T, unscaled, on the current
    stream.  D is overwritten (the reference accumulates into a zeroed D)."""
    tm, tn, tk = PROJECT_TILES[project]
    if m % tm or n % tn or k % tk:
        raise AsyncGemmShapeError(
            f"Either m, n or k is not divisible by the corresponding WARPTILE_ : {m}, {n}, {k}")
    ptr = lambda t: t if isinstance(t, int) else t.data_ptr()  # noqa: E731
    dev = next((t.device for t in (A, B, D) if isinstance(t, torch.Tensor)), torch.device("cuda"))
    if isinstance(D, torch.Tensor):
        assert D.dtype == torch.float32
    with torch.cuda.device(dev):
        code = lib().rdb_dense_gemm_fp8_f32(ptr(A), ptr(B), ptr(D), m, n, k, _stream(dev))
    check(code, "rdb_dense_gemm_fp8_f32")
