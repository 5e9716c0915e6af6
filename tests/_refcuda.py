"""Loader for the reference's own CUDA kernels (oracle/_ref/*.cubin, built unmodified from the reference tree
by `make -C oracle ref`). Test infrastructure: a second checker beside the CPU oracle. Uses the CUDA driver
API through ctypes on the context torch has made current."""
import ctypes as C
import os

import torch

REF_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref")


def available() -> bool:
    return all(os.path.exists(os.path.join(REF_DIR, f)) for f in ("kernels.cubin", "kivi_attn.cubin", "score_reduce.cubin"))


class RefModule:
    def __init__(self, cubin: str):
        torch.cuda.init()
        torch.zeros(1, device="cuda")   # make the primary context current on this thread
        self.cu = C.CDLL("libcuda.so.1")
        self.mod = C.c_void_p()
        rc = self.cu.cuModuleLoad(C.byref(self.mod), os.path.join(REF_DIR, cubin).encode())
        if rc != 0:
            raise RuntimeError(f"cuModuleLoad({cubin}) failed: {rc}")

    def launch(self, name: str, grid, block, smem: int, args) -> None:
        """args: list of ctypes scalars (c_void_p for device pointers, c_int, c_float)."""
        fn = C.c_void_p()
        rc = self.cu.cuModuleGetFunction(C.byref(fn), self.mod, name.encode())
        if rc != 0:
            raise RuntimeError(f"cuModuleGetFunction({name}) failed: {rc}")
        params = (C.c_void_p * len(args))(*[C.cast(C.pointer(a), C.c_void_p) for a in args])
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        rc = self.cu.cuLaunchKernel(fn, *[C.c_uint(g) for g in grid], *[C.c_uint(b) for b in block], C.c_uint(smem), stream,
                                    params, None)
        if rc != 0:
            raise RuntimeError(f"cuLaunchKernel({name}) failed: {rc}")


def ptr(t) -> C.c_void_p:
    return C.c_void_p(0 if t is None else t.data_ptr())
