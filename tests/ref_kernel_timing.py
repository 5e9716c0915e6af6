"""Times the reference's own CUDA kernels (oracle/_ref/*.cubin, built unmodified by `make -C oracle ref`) on this
GPU with the reference's launch shapes, beside this library's prefill. Run by hand: python tests/ref_kernel_timing.py"""
import sys, ctypes as C
import os
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import numpy as np, torch
from tests import _refcuda as ref
from argus_engine_b200 import B200Backend, workloads as wl
from argus_engine_b200.kivi_cache import KiviDeviceCache
be = B200Backend(0)
def tm(fn, n=10):
    for _ in range(2): fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(n): fn()
    b.record(); torch.cuda.synchronize()
    return a.elapsed_time(b) / n
m = ref.RefModule("kernels.cubin")
# C1
hq, hkv, d, T = 32, 8, 64, 2048
q = torch.randn(hq, d, device="cuda"); k = torch.randn(hkv, T, d, device="cuda").half(); v = torch.randn(hkv, T, d, device="cuda").half(); o = torch.zeros(hq, d, device="cuda")
f = lambda: m.launch("attention_gen_f16kv_naive", (hq,1,1), (256,1,1), T*4, [ref.ptr(q), ref.ptr(k), ref.ptr(v), ref.ptr(o), C.c_int(hq), C.c_int(hkv), C.c_int(d), C.c_int(T), C.c_int(T), C.c_void_p(0), C.c_int(0)])
print("ref decode C1 (T=2048,D=64): %.1f us" % (tm(f, 50) * 1e3))
# C2: loop of 16 sequences
lens = wl.config2_lengths(); d = 128
qs = torch.randn(16, hq, d, device="cuda"); ks = [torch.randn(hkv, t, d, device="cuda").half() for t in lens]; vs = [torch.randn(hkv, t, d, device="cuda").half() for t in lens]; o = torch.zeros(16, hq, d, device="cuda")
def f2():
    for i, t in enumerate(lens):
        m.launch("attention_gen_f16kv_naive", (hq,1,1), (256,1,1), t*4, [ref.ptr(qs[i]), ref.ptr(ks[i]), ref.ptr(vs[i]), ref.ptr(o[i]), C.c_int(hq), C.c_int(hkv), C.c_int(d), C.c_int(t), C.c_int(t), C.c_void_p(0), C.c_int(0)])
t2 = tm(f2, 5); by = sum(lens) * hkv * d * 4
print("ref decode C2 (16 launches): %.1f us = %.0f GB/s algorithmic" % (t2 * 1e3, by / t2 / 1e6))
# C3: one sequence q4
mk = ref.RefModule("kivi_attn.cubin")
T = 32768
c = KiviDeviceCache(be, 8, 128, T, 128, 4); c.update(torch.randn(T, 8, 128, device="cuda"), torch.randn(T, 8, 128, device="cuda"))
q = torch.randn(32, 128, device="cuda"); o = torch.zeros(32, 128, device="cuda"); s = torch.zeros(32, T, device="cuda")
f3 = lambda: mk.launch("kernel_attn_gen_kivi_q4", (32,1,1), (64,1,1), 256, [ref.ptr(q), ref.ptr(c.qk), ref.ptr(c.qv), ref.ptr(c.res_k), ref.ptr(c.res_v), ref.ptr(o), ref.ptr(s), C.c_int(32), C.c_int(8), C.c_int(128), C.c_int(c.q_tokens), C.c_int(c.res_pos), C.c_int(128), C.c_float(0.0884), C.c_int(T), C.c_int(1)])
t3 = tm(f3, 3)
print("ref kivi q4 one sequence T=32768: %.1f us (x8 sequences = %.1f ms)" % (t3 * 1e3, t3 * 8))
# C4 reduced
B, S = 1, 1024
q = torch.randn(B, S, 32, 128, device="cuda"); k = torch.randn(B, 8, S, 128, device="cuda").half(); v = torch.randn(B, 8, S, 128, device="cuda").half(); o = torch.zeros(B, S, 32, 128, device="cuda")
f4 = lambda: m.launch("flash_attn_prefill_f16kv_dk128", (S // 32, 32 * B, 1), (32,1,1), 0, [ref.ptr(q), ref.ptr(k), ref.ptr(v), ref.ptr(o), C.c_int(32), C.c_int(8), C.c_int(S), C.c_int(S), C.c_int(S), C.c_int(B)])
t4 = tm(f4, 3); fl = wl.prefill_flops(B, S, S, 32, 128)
print("ref prefill B=1 S=1024: %.3f ms = %.2f TFLOP/s" % (t4, fl / t4 / 1e9))
f5 = lambda: be.flash_attention_prefill(q, k, v, o, 32, 8, S, S, 128, S, B, True)
t5 = tm(f5, 10)
print("ours prefill B=1 S=1024 (F32 Q/O mode): %.3f ms = %.1f TFLOP/s" % (t5, fl / t5 / 1e9))
