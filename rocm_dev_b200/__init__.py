"""B200-native (sm_100a) FP8 GEMM family, sum-reduce and FP8-encoded allreduce.

Host-side mirror of the reference project's launcher interface over a C ABI
(include/rocm_dev_b200.h).  PyTorch is used for device memory and streams only.
"""
from ._lib import LibraryMissing, RdbError, lib, status_string  # noqa: F401
from .allreduce import Fp8AllReduce, LocalRanks, quantize_blocks128, shard_groups  # noqa: F401
from .async_gemm import AsyncGemmShapeError, async_gemm, dense_gemm_fp8  # noqa: F401
from .reduce import globs, globs_n, tiled_sum_reduce  # noqa: F401
from .sparse_gemm import load_2of4, pack_2of4, prune_2of4, save_2of4, sparse_gemm_fp8, sparse_gemm_fp8_grouped  # noqa: F401
from .skinny_gemm import (  # noqa: F401
    OVERLAP_PRIOR_KERNEL,
    HFRK_skinny_gemm,
    SkinnyGemmReturnCode,
    skinny_gemm,
    skinny_gemm_fastpath,
    skinny_gemm_fp8,
    skinny_gemm_fp8_grouped,
    skinny_gemm_fp8_host,
    skinny_gemm_grouped_plan,
    skinny_gemm_fp8_tuned,
)
