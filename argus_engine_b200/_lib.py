"""ctypes binding of ``include/argus_b200.h`` (the same declarations a cgo/Rust FFI stub would carry)."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libargus_b200.so")


class ArgusB200Error(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"argus_b200 error {code}: {msg}")
        self.code = code


class Seq(C.Structure):
    _fields_ = [("k", C.c_void_p), ("v", C.c_void_p), ("seq_len", C.c_int64), ("head_stride", C.c_int64),
                ("pos_stride", C.c_int64)]


class DecodeExtrasC(C.Structure):
    _fields_ = [("scores", C.c_void_p), ("head_scores", C.c_void_p), ("flat_scores", C.c_void_p),
                ("lse", C.c_void_p), ("scores_host", C.c_void_p), ("score_stride", C.c_int64)]


_lib = None


def load_library() -> C.CDLL:
    """Load the CUDA library; fails loudly when it has not been built (no fallback exists)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: run `python -m argus_engine_b200.build` "
                          "(or __graft_entry__.build()) first; there is no CPU fallback")
    lib = C.CDLL(LIB_PATH)
    vp, i32, i64 = C.c_void_p, C.c_int, C.c_int64
    lib.argus_b200_create.argtypes = [i32, C.c_size_t, C.POINTER(vp)]
    lib.argus_b200_destroy.argtypes = [vp]
    lib.argus_b200_destroy.restype = None
    lib.argus_b200_last_error.argtypes = [vp]
    lib.argus_b200_last_error.restype = C.c_char_p
    lib.argus_b200_launch_count.argtypes = [vp]
    lib.argus_b200_launch_count.restype = C.c_uint64
    lib.argus_b200_attention_gen.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, i64, i32, i64, i64,
                                             C.POINTER(DecodeExtrasC)]
    lib.argus_b200_attention_gen_batched.argtypes = [vp, vp, vp, C.POINTER(Seq), i32, vp, i32, i32, i32, i32,
                                                     C.POINTER(DecodeExtrasC)]
    _lib = lib
    return lib
