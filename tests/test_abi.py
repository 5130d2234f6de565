"""CPU tests: the C-ABI library loads without a GPU and exports every symbol
the public header declares."""
import ctypes
import os
import re

import rocm_dev_b200
from rocm_dev_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "rocm_dev_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rdb_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_loads():
    assert os.path.exists(build.build())
    assert b"sm_100a" in rocm_dev_b200.lib().rdb_version()


def test_every_declared_symbol_is_exported_and_bound():
    names = _declared()
    assert "rdb_skinny_gemm_fp8" in names
    handle = ctypes.CDLL(build.LIB_PATH)
    for n in names:
        assert hasattr(handle, n), f"{n} declared in the header but not exported"
    assert sorted(_lib.exported_symbols()) == names, "python binding table and header disagree"


def test_status_strings():
    assert rocm_dev_b200.status_string(0) == "success"
    assert "not even" in rocm_dev_b200.status_string(2)
    assert "timed out" in rocm_dev_b200.status_string(10)


def test_return_codes_keep_reference_numbering():
    from rocm_dev_b200 import SkinnyGemmReturnCode as R
    assert [R.SUCCESS, R.M_ABOVE_WARPTILE_M, R.N_NOT_EVEN, R.K_NOT_DIVISIBLE_BY_WARPTILE_K, R.TOO_MANY_WARPS,
            R.QSIZE_TOO_SMALL, R.INVALID_CONFIG] == list(range(7))
