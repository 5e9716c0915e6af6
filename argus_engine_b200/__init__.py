"""B200 (sm_100a) attention path for argus-engine: a C-ABI CUDA library and a thin Python mirror of the
reference's backend interface, used by the tests and the benchmark.

The CUDA library is the product; there is no CPU fallback. Importing this package does not need a GPU,
but every compute call does, and raises if ``libargus_b200.so`` is missing.
"""
from ._lib import LIB_PATH, ArgusB200Error, load_library  # noqa: F401
from .backend import B200Backend, DecodeExtras  # noqa: F401

__all__ = ["B200Backend", "DecodeExtras", "ArgusB200Error", "load_library", "LIB_PATH"]
