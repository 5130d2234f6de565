"""ctypes binding of the C ABI declared in include/rocm_dev_b200.h.

There is no fallback: if the shared library is missing the import of any
operator fails with an error that says how to build it.
"""
from __future__ import annotations

import ctypes as C
import os

from .build import LIB_PATH

_lib = None

u8p = C.c_void_p
f32p = C.c_void_p
vp = C.c_void_p
i = C.c_int

_SIGNATURES = {
    "rdb_status_string": (C.c_char_p, [i]),
    "rdb_device_status": (i, []),
    "rdb_version": (C.c_char_p, []),
    "rdb_set_wait_budget_ns": (i, [C.c_ulonglong]),
    "rdb_skinny_gemm_fp8": (i, [u8p, u8p, f32p, f32p, vp, i, i, i, i, vp]),
    "rdb_skinny_gemm_fp8_host": (i, [u8p, u8p, f32p, f32p, vp, i, i, i, i, vp]),
    "rdb_skinny_gemm_fp8_hinted": (i, [u8p, u8p, f32p, f32p, vp, i, i, i, i, i, i, i, i, i, i, i, i, vp]),
    "rdb_skinny_gemm_plan": (i, [i, i, i, i, vp, vp, vp]),
    "rdb_tuning_table_load": (i, [C.c_char_p]),
    "rdb_tuning_table_set_skinny": (i, [i, i, i, i, i, i]),
    "rdb_tuning_table_set_dense": (i, [i, i, i, i, i]),
    "rdb_tuning_table_clear": (i, []),
    "rdb_tuning_table_size": (i, []),
    "rdb_skinny_gemm_max_clusters": (i, [i, i, i]),
    "rdb_skinny_gemm_trace": (i, [vp, i, i]),
    "rdb_skinny_gemm_fp8_grouped": (i, [vp, i, C.c_uint, vp]),
    "rdb_skinny_gemm_grouped_plan": (i, [vp, i, i, vp, vp]),
    "rdb_skinny_gemm_grouped_trace": (i, [vp]),
    "rdb_skinny_gemm_fp8_tuned": (i, [u8p, u8p, f32p, f32p, vp, i, i, i, i, i, i, i, C.c_uint, vp]),
    "rdb_dense_gemm_fp8": (i, [u8p, u8p, f32p, f32p, vp, i, i, i, vp]),
    "rdb_dense_gemm_fp8_tuned": (i, [u8p, u8p, f32p, f32p, vp, i, i, i, i, i, vp]),
    "rdb_dense_gemm_fp8_f32": (i, [u8p, u8p, vp, i, i, i, vp]),
    "rdb_sparse_gemm_fp8": (i, [u8p, u8p, u8p, f32p, f32p, vp, i, i, i, vp]),
    "rdb_sparse_gemm_fp8_tuned": (i, [u8p, u8p, u8p, f32p, f32p, vp, i, i, i, i, vp]),
    "rdb_sparse_gemm_trace": (i, [vp, i]),
    "rdb_sparse_gemm_fp8_grouped": (i, [vp, i, C.c_uint, vp]),
    "rdb_sparse_gemm_fp8_flags": (i, [u8p, u8p, u8p, f32p, f32p, vp, i, i, i, i, C.c_uint, vp]),
    "rdb_sparse_meta_bytes": (C.c_size_t, [i, i]),
    "rdb_sparse_pack_2of4": (i, [vp, i, i, vp, vp]),
    "rdb_sparse_file_write": (i, [C.c_char_p, vp, vp, C.c_float, i, i]),
    "rdb_sparse_file_pack_and_write": (i, [C.c_char_p, vp, C.c_float, i, i]),
    "rdb_sparse_file_info": (i, [C.c_char_p, vp, vp, vp]),
    "rdb_sparse_file_read": (i, [C.c_char_p, vp, C.c_size_t, vp, C.c_size_t]),
    "rdb_tiled_sum_reduce": (i, [vp, vp, vp, i, i, i, vp]),
    "rdb_globs": (i, [vp, vp]),
    "rdb_globs_n": (i, [vp, i, i, i, vp]),
    "rdb_ar_workspace_bytes": (C.c_size_t, [i, C.c_size_t]),
    "rdb_ar_workspace_alloc": (i, [C.c_size_t, C.POINTER(C.c_void_p)]),
    "rdb_ar_workspace_free": (i, [vp]),
    "rdb_ar_ipc_export": (i, [vp, C.c_char_p]),
    "rdb_ar_ipc_import": (i, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "rdb_ar_ipc_close": (i, [vp]),
    "rdb_ar_create": (i, [i, i, C.POINTER(C.c_void_p), C.c_size_t, C.POINTER(C.c_void_p)]),
    "rdb_ar_destroy": (i, [vp]),
    "rdb_ar_set_multicast": (i, [vp, vp]),
    "rdb_ar_set_trace": (i, [vp, vp]),
    "rdb_ar_register_buffers": (i, [vp, C.POINTER(C.c_void_p), C.c_size_t]),
    "rdb_ar_set_device_epoch": (i, [vp, i]),
    "rdb_ar_allreduce": (i, [vp, vp, vp, C.c_size_t, i, vp]),
    "rdb_ar_result": (C.c_void_p, [vp]),
    "rdb_skinny_gemm_fp8_allreduce": (i, [vp, vp, vp, vp]),
    "rdb_skinny_gemm_fp8_allreduce_begin": (i, [vp, vp, vp]),
    "rdb_skinny_gemm_fp8_allreduce_finish": (i, [vp, vp, vp]),
    "rdb_ar_begin_call": (i, [vp]),
    "rdb_ar_phase": (i, [vp, i, i, vp, vp, C.c_size_t, i, vp]),
    "rdb_debug_division_mismatches": (i, [vp, i, vp, vp]),
    "rdb_quantize_per_tensor": (i, [vp, vp, vp, C.c_size_t, vp]),
    "rdb_quantize_blocks128": (i, [vp, vp, vp, C.c_size_t, vp]),
    "rdb_globs_n_noalloc": (i, [vp, i, i, i, vp]),
    "rdb_noalloc_status": (i, []),
}


class LibraryMissing(RuntimeError):
    pass


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise LibraryMissing(
                f"{LIB_PATH} not found: build it with `python -m rocm_dev_b200.build` "
                "(there is no CPU or PyTorch fallback)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def exported_symbols() -> list[str]:
    return list(_SIGNATURES)


def status_string(code: int) -> str:
    return lib().rdb_status_string(int(code)).decode()


class RdbError(RuntimeError):
    def __init__(self, code: int, where: str):
        self.code = int(code)
        super().__init__(f"{where}: status {code} ({status_string(code)})")


def check(code: int, where: str) -> None:
    if code != 0:
        raise RdbError(code, where)
