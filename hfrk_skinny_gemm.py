"""``import hfrk_skinny_gemm`` - the module name the reference's torch extension
is built under (projects/skinny_gemm/setup.py:12-16 in the reference project)
with the one class it exports (skinny_gemm_binding.cu:64-104).  Here the class
is the ctypes-backed mirror over librocm_dev_b200.so; there is nothing to
compile with ``setup.py``."""
from rocm_dev_b200.skinny_gemm import HFRK_skinny_gemm  # noqa: F401

__all__ = ["HFRK_skinny_gemm"]
