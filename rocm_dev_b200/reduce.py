"""Host side of tiled_sum_reduce and the grid-barrier probe.

Reference interface (paths within the reference project):
``tiled_sum_reduce(A, B, D, b, m, n)`` - projects/tiled_sum_reduce/src.cu:52-73
and projects/tiled_sum_reduce_async/src.cu:179-200; ``globs(D)`` -
projects/global_sync/src.cu:15-27.
"""
from __future__ import annotations

import torch

from ._lib import check, lib


def _ptr(t):
    return t if isinstance(t, int) else t.data_ptr()


def _dev(*ts):
    return next((t.device for t in ts if isinstance(t, torch.Tensor)), torch.device("cuda"))


def tiled_sum_reduce(A, B, D, b: int, m: int, n: int) -> None:
    """D[m,n] = sum_b (A[b] + B[b]) in fp32 on the current stream."""
    dev = _dev(A, B, D)
    with torch.cuda.device(dev):
        check(lib().rdb_tiled_sum_reduce(_ptr(A), _ptr(B), _ptr(D), b, m, n, torch.cuda.current_stream(dev).cuda_stream),
              "rdb_tiled_sum_reduce")


def globs(D) -> None:
    """The reference's probe: 2 blocks x 64 threads around one grid barrier."""
    dev = _dev(D)
    with torch.cuda.device(dev):
        check(lib().rdb_globs(_ptr(D), torch.cuda.current_stream(dev).cuda_stream), "rdb_globs")


def globs_n(D, blocks: int, threads: int = 64, rounds: int = 1) -> None:
    dev = _dev(D)
    with torch.cuda.device(dev):
        check(lib().rdb_globs_n(_ptr(D), blocks, threads, rounds, torch.cuda.current_stream(dev).cuda_stream),
              "rdb_globs_n")
