"""Second checker: the reference's OWN CUDA kernels (compiled unmodified into oracle/_ref/*.cubin) run on the
same inputs as this library's kernels, launched with the reference's launch shapes
(engine/src/backend/cuda_pc.rs:1793-1800,868-877; crates/techniques/kivi/src/gpu_kivi_cuda.rs:29,197-206;
crates/techniques/attn-score/src/gpu_reduce_cuda.rs:110-111). Skipped when the cubins are absent."""
import ctypes as C

import numpy as np
import pytest
import torch

from argus_engine_b200 import workloads as wl
from tests import _refcuda as ref
from tests._kivi import pack_with_oracle

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref.available(), reason="oracle/_ref cubins not built")]


@pytest.fixture(scope="module")
def be():
    from argus_engine_b200 import B200Backend

    b = B200Backend(0)
    yield b
    b.close()


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("T,hq,hkv,d", [(2048, 32, 8, 64), (5000, 32, 8, 128), (777, 8, 2, 128)])
def test_decode_matches_reference_kernel(be, T, hq, hkv, d):
    """attention_gen_f16kv_naive (engine/src/backend/cuda_pc/kernels.cu:471-540), incl. its score export.
    The first shape is the single short decode of the benchmark set (Hq=32, Hkv=8, D=64, T=2048)."""
    case = wl.decode_case(0, [T], hq, hkv, d)
    q, k, v = _dev(case.q[0]), _dev(case.k[0]), _dev(case.v[0])
    want, want_s = torch.zeros(hq, d, device="cuda"), torch.zeros(hq, T, device="cuda")
    m = ref.RefModule("kernels.cubin")
    m.launch("attention_gen_f16kv_naive", (hq, 1, 1), (256, 1, 1), T * 4,
             [ref.ptr(q), ref.ptr(k), ref.ptr(v), ref.ptr(want), C.c_int(hq), C.c_int(hkv), C.c_int(d), C.c_int(T), C.c_int(T),
              ref.ptr(want_s), C.c_int(T)])
    got, got_s = torch.zeros(hq, d, device="cuda"), torch.zeros(hq, T, device="cuda")
    be.attention_gen(q, k, v, got, hq, hkv, d, T, scores_out=got_s)
    torch.cuda.synchronize()
    np.testing.assert_allclose(got.cpu().numpy(), want.cpu().numpy(), atol=2e-3, rtol=1e-2)
    np.testing.assert_allclose(got_s.cpu().numpy(), want_s.cpu().numpy(), atol=1e-7, rtol=1e-2)


@pytest.mark.parametrize("bits,name", [(2, "kernel_attn_gen_kivi_q2"), (4, "kernel_attn_gen_kivi_q4"), (8, "kernel_attn_gen_kivi_q8")])
def test_kivi_matches_reference_kernel(be, bits, name):
    """kernel_attn_gen_kivi_q{2,4,8} (crates/techniques/kivi/src/kivi_attn.cu:34,220,403)."""
    hq, hkv, d, T = 16, 4, 128, 128 * 4 + 50
    case = pack_with_oracle(wl.kivi_source(bits, [T], hq, hkv, d, 128, bits))
    q, qk, qv = _dev(case.q[0]), _dev(case.qk[0]), _dev(case.qv[0])
    rk, rv = _dev(case.res_k[0]), _dev(case.res_v[0])
    scale = float(1 / np.sqrt(d))
    want, want_s = torch.zeros(hq, d, device="cuda"), torch.zeros(hq, T, device="cuda")
    m = ref.RefModule("kivi_attn.cubin")
    m.launch(name, (hq, 1, 1), (64, 1, 1), 256,
             [ref.ptr(q), ref.ptr(qk), ref.ptr(qv), ref.ptr(rk), ref.ptr(rv), ref.ptr(want), ref.ptr(want_s), C.c_int(hq),
              C.c_int(hkv), C.c_int(d), C.c_int(case.q_tokens[0]), C.c_int(case.res_tokens[0]), C.c_int(128),
              C.c_float(scale), C.c_int(T), C.c_int(1)])
    got = torch.zeros(hq, d, device="cuda")
    got_s = torch.zeros(hq, T)
    assert be.attention_gen_quant(q, qk, qv, rk, rv, got, hq, hkv, d, case.q_tokens[0], case.res_tokens[0], 128, scale, bits,
                                  scores_out=got_s) == 0
    torch.cuda.synchronize()
    np.testing.assert_allclose(got.cpu().numpy(), want.cpu().numpy(), atol=2e-3, rtol=1e-2)
    np.testing.assert_allclose(got_s.numpy(), want_s.cpu().numpy(), atol=1e-7, rtol=1e-2)


def test_score_reduce_matches_reference_kernel(be):
    """kernel_score_fused_reduce / _per_layer (crates/techniques/attn-score/src/score_reduce.cu:13-91)."""
    L, hq, hkv, max_seq, T = 4, 32, 8, 900, 777
    s = torch.rand(L, hq, max_seq, device="cuda")
    imp0, himp0, lf0 = torch.rand(max_seq, device="cuda"), torch.rand(hkv * max_seq, device="cuda"), torch.rand(L * max_seq, device="cuda")
    want = [imp0.clone(), himp0.clone(), lf0.clone()]
    got = [imp0.clone(), himp0.clone(), lf0.clone()]
    m = ref.RefModule("score_reduce.cubin")
    grid = ((T + 63) // 64, 1, 1)
    m.launch("kernel_score_fused_reduce", grid, (64, 1, 1), 0,
             [ref.ptr(s), ref.ptr(want[0]), ref.ptr(want[1]), C.c_float(0.5), C.c_int(L), C.c_int(hq), C.c_int(hkv), C.c_int(T),
              C.c_int(max_seq), C.c_int(max_seq)])
    m.launch("kernel_score_fused_reduce_per_layer", grid, (64, 1, 1), 0,
             [ref.ptr(s), ref.ptr(want[2]), C.c_float(0.5), C.c_int(L), C.c_int(hq), C.c_int(T), C.c_int(max_seq), C.c_int(max_seq)])
    assert be.score_reduce(s, got[0], got[1], 0.5, L, hq, hkv, T, max_seq, max_seq) == 0
    assert be.score_reduce_per_layer(s, got[2], 0.5, L, hq, hkv, T, max_seq, max_seq) == 0
    torch.cuda.synchronize()
    for g, w in zip(got, want):   # decay 0.5 is exact in either rounding order, so the results are bit-identical
        assert torch.equal(g, w)
    # A non-dyadic decay: this library rounds the product and the sum separately, like the CPU producer; the reference
    # kernel as nvcc builds it by default contracts them into one fused multiply-add, so the two may differ by an ulp.
    m.launch("kernel_score_fused_reduce", grid, (64, 1, 1), 0,
             [ref.ptr(s), ref.ptr(want[0]), ref.ptr(want[1]), C.c_float(0.9), C.c_int(L), C.c_int(hq), C.c_int(hkv), C.c_int(T),
              C.c_int(max_seq), C.c_int(max_seq)])
    assert be.score_reduce(s, got[0], got[1], 0.9, L, hq, hkv, T, max_seq, max_seq) == 0
    torch.cuda.synchronize()
    for g, w in zip(got[:2], want[:2]):
        assert torch.allclose(g, w, rtol=3e-7, atol=0)


@pytest.mark.parametrize("S,T", [(256, 256), (100, 300)])
def test_prefill_matches_reference_kernel(be, S, T):
    """flash_attn_prefill_f16kv_dk128 (engine/src/backend/cuda_pc/kernels.cu:691-816,825): F32 Q/O, F16 K/V."""
    B, hq, hkv, d, cap = 2, 8, 2, 128, T + 4
    case = wl.prefill_case(21, B, S, T, hq, hkv, d, cap=cap, dtype="f16")
    q = _dev(case.q)
    k, v = _dev(case.k).half(), _dev(case.v).half()
    want = torch.zeros(B, S, hq, d, device="cuda")
    m = ref.RefModule("kernels.cubin")
    m.launch("flash_attn_prefill_f16kv_dk128", ((S + 31) // 32, hq * B, 1), (32, 1, 1), 0,
             [ref.ptr(q), ref.ptr(k), ref.ptr(v), ref.ptr(want), C.c_int(hq), C.c_int(hkv), C.c_int(S), C.c_int(T), C.c_int(cap),
              C.c_int(B)])
    got = torch.zeros(B, S, hq, d, device="cuda")
    assert be.flash_attention_prefill(q, k, v, got, hq, hkv, S, T, d, cap, B, True)
    torch.cuda.synchronize()
    np.testing.assert_allclose(got.cpu().numpy(), want.cpu().numpy(), atol=2e-3, rtol=1e-2)


def _median_us(fn, n=10):
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
    for a, b in ev:
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    return sorted(a.elapsed_time(b) for a, b in ev)[n // 2] * 1e3


def test_faster_than_the_reference_kernels_on_the_same_gpu(be, capsys):
    """The reference's own CUDA kernels with the reference's launch shapes (engine/src/backend/cuda_pc.rs:1793-1800,
    crates/techniques/kivi/src/gpu_kivi_cuda.rs:197-206) timed beside this library on the same inputs: the single short
    decode (T=2048, D=64) and one KIVI Q4 sequence of 32 768 tokens. Prints the four times (run with -s to see them)."""
    from argus_engine_b200.kivi_cache import KiviDeviceCache

    hq, hkv, d, T = 32, 8, 64, 2048
    case = wl.decode_case(0, [T], hq, hkv, d)
    q, k, v = _dev(case.q[0]), _dev(case.k[0]), _dev(case.v[0])
    o = torch.zeros(hq, d, device="cuda")
    m = ref.RefModule("kernels.cubin")
    ref_decode = _median_us(lambda: m.launch(
        "attention_gen_f16kv_naive", (hq, 1, 1), (256, 1, 1), T * 4,
        [ref.ptr(q), ref.ptr(k), ref.ptr(v), ref.ptr(o), C.c_int(hq), C.c_int(hkv), C.c_int(d), C.c_int(T), C.c_int(T),
         C.c_void_p(0), C.c_int(0)]), 20)
    our_decode = _median_us(lambda: be.attention_gen(q, k, v, o, hq, hkv, d, T), 20)

    hq, hkv, d, T = 32, 8, 128, 32768
    gen = torch.Generator(device="cuda").manual_seed(5)
    cache = KiviDeviceCache(be, hkv, d, T, 128, 4)
    cache.update(torch.randn(T, hkv, d, device="cuda", generator=gen), torch.randn(T, hkv, d, device="cuda", generator=gen))
    q = torch.randn(hq, d, device="cuda", generator=gen)
    o_ref, o_our = torch.zeros(hq, d, device="cuda"), torch.zeros(hq, d, device="cuda")
    s_ref = torch.zeros(hq, T, device="cuda")
    scale = float(1 / np.sqrt(d))
    mk = ref.RefModule("kivi_attn.cubin")
    ref_kivi = _median_us(lambda: mk.launch(
        "kernel_attn_gen_kivi_q4", (hq, 1, 1), (64, 1, 1), 256,
        [ref.ptr(q), ref.ptr(cache.qk), ref.ptr(cache.qv), ref.ptr(cache.res_k), ref.ptr(cache.res_v), ref.ptr(o_ref),
         ref.ptr(s_ref), C.c_int(hq), C.c_int(hkv), C.c_int(d), C.c_int(cache.q_tokens), C.c_int(cache.res_pos), C.c_int(128),
         C.c_float(scale), C.c_int(T), C.c_int(1)]), 3)
    seq = [cache.seq()]
    our_kivi = _median_us(lambda: be.kivi_attention_batched(q[None], seq, o_our[None], hq, hkv, d, 128, 4, scale), 10)
    torch.cuda.synchronize()
    np.testing.assert_allclose(o_our.cpu().numpy(), o_ref.cpu().numpy(), atol=2e-3, rtol=1e-2)
    with capsys.disabled():
        print(f"\n[reference kernels on this GPU] decode T=2048 D=64: reference {ref_decode:.1f} us, library {our_decode:.1f} us | "
              f"KIVI Q4 one sequence T=32768: reference {ref_kivi / 1e3:.2f} ms, library {our_kivi:.1f} us")
    assert our_decode * 5 < ref_decode
    assert our_kivi * 50 < ref_kivi
