"""GPU parity of the split-KV F16 decode kernel against the CPU oracle, through the C ABI.

Tolerances are the ones the task states for attention outputs and H2O scores: max-abs 2e-3 / rel 1e-2
against the F32 reference (np.allclose form |a-b| <= atol + rtol*|b|). Score probabilities are O(1/T),
so they are checked with the relative bound and a tiny absolute floor.
"""
import numpy as np
import pytest
import torch

from argus_engine_b200 import workloads as wl
from oracle import oracle as orc

pytestmark = pytest.mark.gpu

OUT_ATOL, OUT_RTOL = 2e-3, 1e-2
P_ATOL, P_RTOL = 1e-7, 1e-2


@pytest.fixture(scope="module")
def be():
    from argus_engine_b200 import B200Backend

    b = B200Backend(0)
    yield b
    b.close()


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _oracle(case, i, head_major=True, scores=False):
    k, v = case.k[i].view(np.uint16), case.v[i].view(np.uint16)
    return orc.attention_gen(case.q[i], k, v, case.hq, case.hkv, case.d, case.lens[i], head_major,
                             want_scores=scores)


def _run_single(be, case, i=0, seq_major=False, scores_stride=None, host_scores=False, lse=False):
    from argus_engine_b200 import DecodeExtras

    k, v = case.k[i], case.v[i]
    if seq_major:
        k, v = (np.ascontiguousarray(a.transpose(1, 0, 2)) for a in (k, v))
    kd, vd, qd = _dev(k), _dev(v), _dev(case.q[i])
    out = torch.full((case.hq, case.d), float("nan"), device="cuda")
    ex = DecodeExtras()
    sc = None
    if scores_stride:
        sc = torch.full((case.hq, scores_stride), -1.0, device="cpu" if host_scores else "cuda")
    if lse:
        ex.lse = torch.zeros(case.hq, device="cuda")
    be.attention_gen(qd, kd, vd, out, case.hq, case.hkv, case.d, case.lens[i], scores_out=sc, extras=ex)
    torch.cuda.synchronize()
    return out.cpu().numpy(), None if sc is None else sc.cpu().numpy(), None if not lse else ex.lse.cpu().numpy()


def test_config1_parity(be):
    """The single short decode of the benchmark set: B=1, Hq=32, Hkv=8, D=64, T=2048, seed 0."""
    case = wl.config1()
    want, _ = _oracle(case, 0)
    got, _, _ = _run_single(be, case)
    np.testing.assert_allclose(got, want, atol=OUT_ATOL, rtol=OUT_RTOL)
    assert np.max(np.abs(got - want)) < 2e-4   # what the hi/lo operand split actually delivers


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("g", [1, 2, 4, 8])
@pytest.mark.parametrize("T", [1, 15, 16, 17, 63, 64, 65, 129, 1000, 2500])
def test_shapes_and_ragged_lengths(be, d, g, T):
    hkv = 2
    case = wl.decode_case(100 + T + d + g, [T], hkv * g, hkv, d, cap_extra=7)
    for a in (case.k[0], case.v[0]):
        a[:, T:, :] = np.nan   # rows past cache_seq_len must never be read into the result
    want, want_p = _oracle(case, 0, scores=True)
    got, got_p, lse = _run_single(be, case, scores_stride=T + 3, lse=True)
    np.testing.assert_allclose(got, want, atol=OUT_ATOL, rtol=OUT_RTOL)
    np.testing.assert_allclose(got_p[:, :T], want_p, atol=P_ATOL, rtol=P_RTOL)
    assert np.all(got_p[:, T:] == -1.0)   # padding of the score rows is left alone
    kf = case.k[0][:, :T].astype(np.float64)
    s = np.einsum("htd,hgd->hgt", kf, case.q[0].reshape(hkv, g, d).astype(np.float64)) / np.sqrt(d)
    want_lse = np.log(np.exp(s - s.max(-1, keepdims=True)).sum(-1)) + s.max(-1)
    np.testing.assert_allclose(lse, want_lse.reshape(-1), atol=1e-3)


@pytest.mark.parametrize("T", [333, 4096])
def test_seq_major_layout(be, T):
    case = wl.decode_case(7, [T], 8, 2, 128)
    want, _ = _oracle(case, 0)
    got, _, _ = _run_single(be, case, seq_major=True)
    np.testing.assert_allclose(got, want, atol=OUT_ATOL, rtol=OUT_RTOL)


def test_host_scores_blocking_readback(be):
    """`scores_out` as a host slice: filled when the call returns (engine/src/backend/cuda_pc.rs:1867-1880)."""
    case = wl.decode_case(11, [777], 8, 2, 64)
    want, want_p = _oracle(case, 0, scores=True)
    got, got_p, _ = _run_single(be, case, scores_stride=800, host_scores=True)
    np.testing.assert_allclose(got, want, atol=OUT_ATOL, rtol=OUT_RTOL)
    np.testing.assert_allclose(got_p[:, :777], want_p, atol=P_ATOL, rtol=P_RTOL)


def test_batched_varlen_with_fused_group_scores(be):
    """The batched decode scaled down (Llama-3-8B head shape, lengths U[64,1500]) incl. an empty sequence."""
    from argus_engine_b200 import DecodeExtras

    lens = wl.config2_lengths(6, 64, 1500) + [0]
    case = wl.decode_case(1, lens, 32, 8, 128)
    B, stride = len(lens), 1536
    qd = _dev(case.q)
    kd = [_dev(a) if a.size else torch.zeros(8, 1, 128, dtype=torch.float16, device="cuda") for a in case.k]
    vd = [_dev(a) if a.size else torch.zeros(8, 1, 128, dtype=torch.float16, device="cuda") for a in case.v]
    out = torch.full((B, 32, 128), float("nan"), device="cuda")
    ex = DecodeExtras(head_scores=torch.zeros(B, 8, stride, device="cuda"),
                      flat_scores=torch.zeros(B, stride, device="cuda"),
                      lse=torch.zeros(B, 32, device="cuda"), score_stride=stride)
    be.attention_gen_batched(qd, kd, vd, lens, out, 32, 8, 128, extras=ex)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    for i, T in enumerate(lens):
        if T == 0:
            assert np.all(got[i] == 0.0) and np.all(np.isneginf(ex.lse[i].cpu().numpy()))
            continue
        want, want_p = _oracle(case, i, scores=True)
        np.testing.assert_allclose(got[i], want, atol=OUT_ATOL, rtol=OUT_RTOL)
        sf = np.zeros(stride, dtype=np.float32)
        sh = np.zeros(8 * stride, dtype=np.float32)
        orc.score_accumulate_layer(want_p, T, 32, 8, stride, sf, sh)
        np.testing.assert_allclose(ex.head_scores[i].cpu().numpy()[:, :T], sh.reshape(8, stride)[:, :T],
                                   atol=P_ATOL, rtol=P_RTOL)
        np.testing.assert_allclose(ex.flat_scores[i].cpu().numpy()[:T], sf[:T], atol=P_ATOL, rtol=P_RTOL)


def test_many_splits_and_determinism(be):
    """Long sequence => many splits merged through the ticket path; two runs are bit-identical."""
    case = wl.decode_case(5, [50000], 16, 2, 128)
    want, _ = _oracle(case, 0)
    a, _, _ = _run_single(be, case)
    b, _, _ = _run_single(be, case)
    np.testing.assert_allclose(a, want, atol=OUT_ATOL, rtol=OUT_RTOL)
    assert np.array_equal(a, b)


@pytest.mark.parametrize("seq_major", [False, True])
def test_f32_kv_cache(be, seq_major):
    """F32 K/V (engine/src/backend.rs:305-313): served through an F16 copy; the oracle reads the F32 values."""
    T, hq, hkv, d = 1500, 16, 4, 128
    rng = np.random.default_rng(8)
    q = rng.standard_normal((hq, d), dtype=np.float32)
    k = rng.standard_normal((hkv, T, d), dtype=np.float32)
    v = rng.standard_normal((hkv, T, d), dtype=np.float32)
    want, _ = orc.attention_gen(q, k, v, hq, hkv, d, T)
    if seq_major:
        k, v = (np.ascontiguousarray(a.transpose(1, 0, 2)) for a in (k, v))
    out = torch.zeros(hq, d, device="cuda")
    be.attention_gen(_dev(q), _dev(k), _dev(v), out, hq, hkv, d, T)
    torch.cuda.synchronize()
    np.testing.assert_allclose(out.cpu().numpy(), want, atol=OUT_ATOL, rtol=OUT_RTOL)


def test_argument_errors(be):
    from argus_engine_b200 import ArgusB200Error

    q = torch.zeros(8, 96, device="cuda")
    k = torch.zeros(2, 16, 96, dtype=torch.float16, device="cuda")
    with pytest.raises(ArgusB200Error) as e:   # head_dim 96 is declined, not faulted
        be.attention_gen(q, k, k, torch.zeros_like(q), 8, 2, 96, 16)
    assert e.value.code == -2
    q = torch.zeros(8, 64, device="cuda")
    k = torch.zeros(2, 16, 64, dtype=torch.float16, device="cuda")
    with pytest.raises(ArgusB200Error) as e:   # 8 query heads over 3 KV heads
        be.attention_gen(q, k, k, torch.zeros_like(q), 8, 3, 64, 16)
    assert e.value.code == -1


@pytest.mark.parametrize("d,page_tokens", [(128, 16), (128, 256), (64, 64)])
def test_paged_cache_is_bit_identical_to_contiguous(be, d, page_tokens):
    """Paged layout option: the same tokens scattered over a shuffled page pool give the same bits as the contiguous
    caches (same split plan, same tile order), outputs and fused score vectors alike, and match the oracle."""
    from argus_engine_b200 import DecodeExtras

    lens = [5000, 333, 16, 4097, 1]
    hq, hkv = 16, 4
    case = wl.decode_case(77 + d, lens, hq, hkv, d)
    B, stride = len(lens), 5008
    ks, vs = [_dev(k) for k in case.k], [_dev(v) for v in case.v]
    out_c = torch.zeros(B, hq, d, device="cuda")
    ex_c = DecodeExtras(head_scores=torch.zeros(B, hkv, stride, device="cuda"), score_stride=stride)
    be.attention_gen_batched(_dev(case.q), ks, vs, lens, out_c, hq, hkv, d, extras=ex_c)
    # pool: every sequence's pages land at random places of one pool
    n_pages = sum((t + page_tokens - 1) // page_tokens for t in lens)
    rng = np.random.default_rng(5)
    perm = rng.permutation(n_pages + 3)
    k_pool = torch.zeros(n_pages + 3, hkv, page_tokens, d, device="cuda", dtype=torch.float16)
    v_pool = torch.zeros_like(k_pool)
    tables, nxt = [], 0
    for i, t in enumerate(lens):
        npg = (t + page_tokens - 1) // page_tokens
        ids = perm[nxt:nxt + npg]
        nxt += npg
        for j, pg in enumerate(ids):
            lo, hi = j * page_tokens, min((j + 1) * page_tokens, t)
            k_pool[pg, :, :hi - lo] = ks[i][:, lo:hi]
            v_pool[pg, :, :hi - lo] = vs[i][:, lo:hi]
        tables.append(torch.from_numpy(ids.astype(np.int32)).cuda())
    out_p = torch.full((B, hq, d), float("nan"), device="cuda")
    ex_p = DecodeExtras(head_scores=torch.zeros(B, hkv, stride, device="cuda"), score_stride=stride)
    be.attention_gen_paged(_dev(case.q), k_pool, v_pool, tables, lens, out_p, hq, extras=ex_p)
    torch.cuda.synchronize()
    assert be.check_status() == 0
    assert torch.equal(out_p, out_c)
    assert torch.equal(ex_p.head_scores, ex_c.head_scores)
    for i in range(B):
        want, _ = _oracle(case, i)
        np.testing.assert_allclose(out_p[i].cpu().numpy(), want, atol=OUT_ATOL, rtol=OUT_RTOL)


@pytest.mark.parametrize("seq_major", [False, True])
def test_decode_step_writes_the_row_and_attends(be, seq_major):
    """argus_b200_decode_step_batched = KV write + attention in one launch: caches and outputs are bit-identical to
    argus_b200_kv_scatter_batched followed by argus_b200_attention_gen_batched, and the output matches the oracle run
    on the F16-rounded new rows. Lengths cover an empty cache, a row that opens a new 16-token tile and ragged ends."""
    hq, hkv, d, cap_extra = 32, 8, 128, 40
    lens = [0, 15, 16, 1000, 4099]            # lengths BEFORE the step
    case = wl.decode_case(77, [t + 1 for t in lens], hq, hkv, d, cap_extra=cap_extra)
    rng = np.random.Generator(np.random.PCG64(78))
    k_new = rng.standard_normal((len(lens), hkv, d), dtype=np.float32)
    v_new = rng.standard_normal((len(lens), hkv, d), dtype=np.float32)

    def caches():
        ks, vs = [], []
        for i in range(len(lens)):
            k, v = case.k[i].copy(), case.v[i].copy()
            k[:, lens[i]:] = np.nan   # the new row's slot and everything behind it hold garbage before the step
            v[:, lens[i]:] = np.nan
            if seq_major:
                k, v = (np.ascontiguousarray(a.transpose(1, 0, 2)) for a in (k, v))
            ks.append(_dev(k))
            vs.append(_dev(v))
        return ks, vs

    q = _dev(case.q)
    ks1, vs1 = caches()
    out1 = torch.full((len(lens), hq, d), float("nan"), device="cuda")
    launches0 = be.launch_count
    be.decode_step_batched(q, _dev(k_new), _dev(v_new), ks1, vs1, lens, out1, hq, hkv, d)
    assert be.launch_count - launches0 == 1
    ks2, vs2 = caches()
    out2 = torch.full((len(lens), hq, d), float("nan"), device="cuda")
    if seq_major:   # the batched KV write takes HeadMajor caches: write through a transposed view of the same memory
        for i in range(len(lens)):
            ks2[i][lens[i]] = _dev(k_new[i]).to(torch.float16)
            vs2[i][lens[i]] = _dev(v_new[i]).to(torch.float16)
    else:
        be.kv_scatter_batched(_dev(k_new), _dev(v_new), ks2, vs2, lens)
    be.attention_gen_batched(q, ks2, vs2, [t + 1 for t in lens], out2, hq, hkv, d)
    torch.cuda.synchronize()
    assert be.check_status() == 0
    assert torch.equal(out1, out2)
    for i, t in enumerate(lens):
        a, b = (ks1[i], ks2[i]), (vs1[i], vs2[i])
        for x, y in (a, b):
            rows_x = x[: t + 1] if seq_major else x[:, : t + 1]
            rows_y = y[: t + 1] if seq_major else y[:, : t + 1]
            assert torch.equal(rows_x.view(torch.int16), rows_y.view(torch.int16))
        kk = case.k[i].copy()
        vv = case.v[i].copy()
        kk[:, t] = k_new[i].astype(np.float16)
        vv[:, t] = v_new[i].astype(np.float16)
        want, _ = orc.attention_gen(case.q[i], kk.view(np.uint16), vv.view(np.uint16), hq, hkv, d, t + 1)
        np.testing.assert_allclose(out1[i].cpu().numpy(), want, atol=OUT_ATOL, rtol=OUT_RTOL)


def test_nan_logit_is_skipped_like_the_cpu_guard(be):
    """What a NaN in the K cache does. The reference's CPU backends turn NaN logits into -inf, i.e. skip the position
    (engine/src/backend/cpu/common.rs:555-584); its CUDA kernel (engine/src/backend/cuda_pc/kernels.cu:471-540) and its
    AVX2 arm have no guard and return NaN rows. This kernel follows the CPU guard for NaN logits: the heads that read the
    NaN row equal the guarded oracle, the exported probability of that position is 0, other KV heads are untouched.
    (The guard's second half, a uniform distribution when NO finite logit is left, is not reproduced: such a head
    returns zeros and lse = -inf, checked below with a NaN in q.)"""
    from argus_engine_b200 import DecodeExtras

    hq, hkv, d, T = 8, 2, 64, 300
    case = wl.decode_case(5, [T], hq, hkv, d)
    k = case.k[0].copy()
    k[1, 17, 3] = np.nan
    out = torch.zeros(hq, d, device="cuda")
    sc = torch.zeros(hq, T, device="cuda")
    be.attention_gen(_dev(case.q[0]), _dev(k), _dev(case.v[0]), out, hq, hkv, d, T, scores_out=sc)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    guarded, guarded_p = orc.attention_gen(case.q[0], k.view(np.uint16), case.v[0].view(np.uint16), hq, hkv, d, T,
                                           want_scores=True, guards=True)
    assert np.isfinite(guarded).all()
    np.testing.assert_allclose(got, guarded, atol=OUT_ATOL, rtol=OUT_RTOL)
    np.testing.assert_allclose(sc.cpu().numpy(), guarded_p, atol=P_ATOL, rtol=P_RTOL)
    g = hq // hkv
    assert (sc[g:, 17] == 0).all()
    unguarded, _ = orc.attention_gen(case.q[0], k.view(np.uint16), case.v[0].view(np.uint16), hq, hkv, d, T)
    assert np.isnan(unguarded[g:]).all()                # the unguarded arms return NaN rows here
    q = case.q[0].copy()
    q[5, 0] = np.nan                                    # every logit of query head 5 is NaN: nothing finite is left
    lse = torch.zeros(hq, device="cuda")
    be.attention_gen(_dev(q), _dev(case.k[0]), _dev(case.v[0]), out, hq, hkv, d, T, extras=DecodeExtras(lse=lse))
    torch.cuda.synchronize()
    assert torch.count_nonzero(out[5]) == 0 and torch.isneginf(lse[5])
    want, _ = orc.attention_gen(case.q[0], case.k[0].view(np.uint16), case.v[0].view(np.uint16), hq, hkv, d, T)
    keep = [h for h in range(hq) if h != 5]
    np.testing.assert_allclose(out.cpu().numpy()[keep], want[keep], atol=OUT_ATOL, rtol=OUT_RTOL)


def test_context_created_inside_the_callers_cuda_context():
    """argus_b200_create_in_context takes the raw CUcontext the engine lends to a plugin factory
    (CudaQuantAttnMakeArgs.cu_context, crates/argus-extension-api/src/lib.rs:2985-2994): the context is pushed for the
    allocations and popped again, and decode through the object works from a thread that has it current."""
    import ctypes as C

    from argus_engine_b200 import B200Backend

    torch.zeros(1, device="cuda")
    cu = C.CDLL("libcuda.so.1")
    cur = C.c_void_p()
    assert cu.cuCtxGetCurrent(C.byref(cur)) == 0 and cur.value
    b = B200Backend(0, cu_context=cur.value)
    after = C.c_void_p()
    assert cu.cuCtxGetCurrent(C.byref(after)) == 0 and after.value == cur.value   # pushed and popped: nothing left behind
    case = wl.decode_case(3, [700], 32, 8, 128)
    want, _ = _oracle(case, 0)
    got, _, _ = _run_single(b, case)
    np.testing.assert_allclose(got, want, atol=OUT_ATOL, rtol=OUT_RTOL)
    b.close()
    with pytest.raises(Exception):
        B200Backend(0, cu_context=0)
