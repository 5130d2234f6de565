"""Host side of the 2:4 structured-sparse FP8 GEMM.

The reference's ``async_gemm_sparse`` (projects/async_gemm_sparse/ in the
reference project) keeps the dense launcher signature ``async_gemm(A, B, D, m,
n, k)`` and contains no pruning or compression; the pruning rule, the
compressed format and the packer here implement the configuration text: keep
the two largest magnitudes of every aligned group of four along K (ties: the
lowest index), quantise per tensor, store the kept bytes plus 2-bit positions.
"""
from __future__ import annotations

import ctypes as C

import torch

from ._lib import check, lib


def prune_2of4(W: torch.Tensor) -> torch.Tensor:
    """Zero all but the two largest-magnitude entries of each group of four
    along the last dimension (ties: lowest index).  CPU or GPU tensor."""
    assert W.shape[-1] % 4 == 0
    g = W.reshape(-1, 4)
    a = g.abs().float()
    # stable descending order keeps the lower index on ties
    order = torch.argsort(a, dim=1, descending=True, stable=True)
    keep = torch.zeros_like(a, dtype=torch.bool)
    keep.scatter_(1, order[:, :2], True)
    return torch.where(keep, g, torch.zeros_like(g)).reshape(W.shape)


def pack_2of4(Wq: torch.Tensor):
    """Wq: [N,K] uint8 e4m3 bytes that are already 2:4 (CPU).  Returns
    (vals [N,K/2] uint8, meta uint8) in the layout the kernel consumes."""
    assert Wq.dtype == torch.uint8 and Wq.dim() == 2 and not Wq.is_cuda
    Wq = Wq.contiguous()
    N, K = Wq.shape
    nbytes = int(lib().rdb_sparse_meta_bytes(N, K))
    if nbytes == 0:
        raise ValueError("K must be a multiple of 256")
    vals = torch.empty((N, K // 2), dtype=torch.uint8)
    meta = torch.empty(nbytes, dtype=torch.uint8)
    check(lib().rdb_sparse_pack_2of4(Wq.data_ptr(), N, K, vals.data_ptr(), meta.data_ptr()), "rdb_sparse_pack_2of4")
    return vals, meta


def save_2of4(path: str, vals: torch.Tensor, meta: torch.Tensor, scale: float) -> None:
    """Writes compressed weights (as returned by ``pack_2of4``) and their
    per-tensor scale as one file (rdb_sparse_file_write)."""
    import ctypes as C
    assert vals.dtype == torch.uint8 and meta.dtype == torch.uint8 and not vals.is_cuda and not meta.is_cuda
    vals, meta = vals.contiguous(), meta.contiguous()
    N, K2 = vals.shape
    check(lib().rdb_sparse_file_write(str(path).encode(), vals.data_ptr(), meta.data_ptr(), C.c_float(float(scale)), N, 2 * K2),
          "rdb_sparse_file_write")


def load_2of4(path: str):
    """Reads a file written by ``save_2of4``: (vals [N,K/2] uint8, meta uint8, scale).
    Raises RdbError for a file that is not of this format, is damaged or does
    not hold a 2:4 selection."""
    import ctypes as C
    n, k, sc = C.c_int(), C.c_int(), C.c_float()
    check(lib().rdb_sparse_file_info(str(path).encode(), C.byref(n), C.byref(k), C.byref(sc)), "rdb_sparse_file_info")
    N, K = n.value, k.value
    vals = torch.empty((N, K // 2), dtype=torch.uint8)
    meta = torch.empty(int(lib().rdb_sparse_meta_bytes(N, K)), dtype=torch.uint8)
    check(lib().rdb_sparse_file_read(str(path).encode(), vals.data_ptr(), vals.numel(), meta.data_ptr(), meta.numel()),
          "rdb_sparse_file_read")
    return vals, meta, sc.value


def sparse_gemm_fp8(A: torch.Tensor, vals: torch.Tensor, meta: torch.Tensor, scale_a: torch.Tensor,
                    scale_b: torch.Tensor, out: torch.Tensor | None = None, split_k: int = 0, flags: int = 0) -> torch.Tensor:
    """D[M,N] = bf16((A . W^T) * scale_a * scale_b) with W given compressed.
    ``flags``: 0 or ``OVERLAP_PRIOR_KERNEL`` (1): the launch may start streaming
    weights while the preceding kernel of the stream drains (that kernel must not
    write the weights)."""
    assert A.is_cuda and vals.is_cuda and meta.is_cuda and A.is_contiguous() and vals.is_contiguous()
    A = A if A.dtype == torch.uint8 else A.view(torch.uint8)
    M, K = A.shape
    N = vals.shape[0]
    assert vals.shape[1] * 2 == K
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=A.device)
    with torch.cuda.device(A.device):
        check(lib().rdb_sparse_gemm_fp8_flags(A.data_ptr(), vals.data_ptr(), meta.data_ptr(), scale_a.data_ptr(),
                                              scale_b.data_ptr(), out.data_ptr(), M, N, K, split_k, flags,
                                              torch.cuda.current_stream(A.device).cuda_stream), "rdb_sparse_gemm_fp8")
    return out


class SparseProblem(C.Structure):
    """``rdb_sparse_problem`` of include/rocm_dev_b200.h."""
    _fields_ = [("A", C.c_void_p), ("Wvals", C.c_void_p), ("Wmeta", C.c_void_p), ("scale_a", C.c_void_p),
                ("scale_b", C.c_void_p), ("D", C.c_void_p), ("M", C.c_int), ("N", C.c_int), ("K", C.c_int)]


def sparse_gemm_fp8_grouped(problems, flags: int = 0) -> int:
    """A list of sparse GEMMs with one batch size in ONE launch
    (rdb_sparse_gemm_fp8_grouped).  ``problems``: up to 8 tuples ``(A, vals,
    meta, scale_a, scale_b, D)`` of device tensors with the meaning of
    ``sparse_gemm_fp8``; all A must have the same number of rows.  Returns the
    status code."""
    arr = (SparseProblem * len(problems))()
    for i, (A, vals, meta, sa, sb, D) in enumerate(problems):
        A = A if A.dtype == torch.uint8 else A.view(torch.uint8)
        M, K = A.shape
        assert vals.shape[1] * 2 == K and D.dtype == torch.bfloat16 and D.is_contiguous() and D.shape == (M, vals.shape[0])
        arr[i] = SparseProblem(A.data_ptr(), vals.data_ptr(), meta.data_ptr(), sa.data_ptr(), sb.data_ptr(), D.data_ptr(),
                               M, vals.shape[0], K)
    dev = problems[0][0].device
    with torch.cuda.device(dev):
        return int(lib().rdb_sparse_gemm_fp8_grouped(arr, len(problems), flags, torch.cuda.current_stream(dev).cuda_stream))
