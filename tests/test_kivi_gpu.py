"""GPU parity of the KIVI path through the C ABI: bit-exact pack/unpack and container kernels, and the
fused dequant+decode kernel against the oracle's F32 view + three-pass attention.

Tolerances: pack/unpack and data movement bit-exact; attention outputs max-abs 2e-3 / rel 1e-2; scores
rel 1e-2 (absolute floor 1e-7).
"""
import numpy as np
import pytest
import torch

from argus_engine_b200 import workloads as wl
from oracle import oracle as orc
from tests._kivi import pack_with_oracle

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


def _adversarial_ring(rng, hkv, rc, d):
    """Values that stress the codec's rounding: .5 ties, constant groups, signed zeros, tiny and huge ranges."""
    x = rng.standard_normal((hkv, rc, d)).astype(np.float32)
    x[0, :, 0] = 3.25                       # constant channel: d == 0
    x[0, :, 1] = np.arange(rc) % 16 + 0.5   # ties at .5 when the scale is 1
    x[0, :, 2] = 0.0                        # all-zero channel (a group mixing +0 and -0 is left out: the sign of
                                            # a zero minimum is unspecified by IEEE minNum, hence by f32::min)
    x[0, :, 3] = rng.standard_normal(rc) * 1e-30
    x[0, :, 4] = rng.standard_normal(rc) * 7e4   # min overflows F16 -> inf in the stored field, like the CPU
    x[0, 0, :] = 1.0                        # constant token for V
    x[0, 1, :32] = np.arange(32) * 0.5      # .5 ties along channels
    return x


@pytest.mark.parametrize("bits", [2, 4, 8])
@pytest.mark.parametrize("d,rc", [(128, 128), (64, 32), (128, 64)])
def test_flush_pack_bit_exact(be, bits, d, rc):
    """KIVI pack: device flush == CPU codec bytes (crates/argus-kv-codec/src/lib.rs), in flush order."""
    hkv = 3
    rng = np.random.default_rng(bits * 100 + d)
    rk, rv = _adversarial_ring(rng, hkv, rc, d), _adversarial_ring(rng, hkv, rc, d)
    c = orc.KiviCache(hkv, d, rc, bits)
    seq = np.ascontiguousarray(rk.transpose(1, 0, 2)), np.ascontiguousarray(rv.transpose(1, 0, 2))
    c.update(*seq)
    c.update(seq[0][:1], seq[1][:1])   # the next write triggers the flush
    want_k, want_v, _, _ = c.export()
    bb = orc.block_bytes(bits)
    pad = 5   # blocks of padding in front: the entry appends at a block offset
    qk = torch.full((want_k.size + pad * bb,), 0xEE, dtype=torch.uint8, device="cuda")
    qv = torch.full((want_v.size + pad * bb,), 0xEE, dtype=torch.uint8, device="cuda")
    be.kivi_flush_pack(_dev(rk), _dev(rv), qk, qv, hkv, d, rc, rc // 32, bits, pad, pad)
    torch.cuda.synchronize()
    for name, got, want in (("K", qk, want_k), ("V", qv, want_v)):
        got = got.cpu().numpy()[pad * bb:]
        bad = np.flatnonzero(got != want)
        assert bad.size == 0, f"{name}: {bad.size} bytes differ, first in block {bad[0] // bb} at byte {bad[0] % bb}: " \
                              f"got {got[bad[0] // bb * bb:(bad[0] // bb + 1) * bb].tolist()} want " \
                              f"{want[bad[0] // bb * bb:(bad[0] // bb + 1) * bb].tolist()}"
    assert np.all(qk.cpu().numpy()[:pad * bb] == 0xEE)


@pytest.mark.parametrize("bits", [2, 4, 8])
def test_container_kernels_round_trip(be, bits):
    """gather_update, dequant_flush and scatter_residual against the oracle's view
    (the round trips of engine/src/bin/test_cuda_quant_attn_device.rs, cases C-E)."""
    hkv, d, rc, T = 2, 64, 64, 64 * 2 + 17
    rng = np.random.default_rng(bits)
    k = rng.standard_normal((T, hkv, d)).astype(np.float32)
    v = rng.standard_normal((T, hkv, d)).astype(np.float32)
    c = orc.KiviCache(hkv, d, rc, bits)
    c.update(k, v)
    qk, qv, rk, rv = c.export()
    vk, vv = orc.kivi_assemble_view(qk, qv, rk, rv, hkv, d, rc, bits, c.q_tokens, c.res_tokens)
    # gather_update: rows land at res_pos.. of the ring, F32 exact
    ring = torch.zeros(hkv, rc, d, device="cuda")
    assert be.gather_update_quant(_dev(k[128:]), ring, hkv, rc, d, T - 128, 0) == 0
    assert np.array_equal(ring.cpu().numpy()[:, :17], rk[:, :17])
    assert be.gather_update_quant(_dev(k[:rc]), ring, hkv, rc, d, rc, 1) == -1   # would overflow the ring
    # dequant_flush + scatter_residual build the F16 SeqMajor view
    attn_k = torch.zeros(T, hkv, d, dtype=torch.float16, device="cuda")
    attn_v = torch.zeros(T, hkv, d, dtype=torch.float16, device="cuda")
    qkd, qvd = _dev(qk), _dev(qv)
    kbpf, vbpf = hkv * (rc // 32) * d, hkv * rc * (d // 32)
    for f in range(2):
        assert be.dequant_flush(qkd, attn_k, hkv, d, rc // 32, f * rc, f * kbpf, bits, True) == 0
        assert be.dequant_flush(qvd, attn_v, hkv, d, rc, f * rc, f * vbpf, bits, False) == 0
    assert be.scatter_residual(_dev(rk), attn_k, hkv, rc, d, 17, 128) == 0
    assert be.scatter_residual(_dev(rv), attn_v, hkv, rc, d, 17, 128) == 0
    torch.cuda.synchronize()
    assert np.array_equal(attn_k.cpu().numpy(), vk.astype(np.float16))
    assert np.array_equal(attn_v.cpu().numpy(), vv.astype(np.float16))


def _oracle_kivi(case, i, scale=None, scores=False):
    hkv, d = case.hkv, case.d
    rk, rv = case.res_k[i].astype(np.float32), case.res_v[i].astype(np.float32)
    vk, vv = orc.kivi_assemble_view(case.qk[i], case.qv[i], rk, rv, hkv, d, case.res_cap, case.bits,
                                    case.q_tokens[i], case.res_tokens[i])
    T = case.q_tokens[i] + case.res_tokens[i]
    q = case.q[i]
    if scale is not None:   # the oracle applies 1/sqrt(D); fold any other scale into q
        q = q * np.float32(scale * np.sqrt(d))
    return orc.attention_gen(q, vk, vv, case.hq, hkv, d, T, head_major=False, want_scores=scores)


@pytest.mark.parametrize("bits", [2, 4, 8])
@pytest.mark.parametrize("d,g", [(128, 4), (64, 8), (128, 1)])
@pytest.mark.parametrize("T", [5, 128, 133, 128 * 3, 128 * 5 + 77])
def test_attention_gen_quant_vs_oracle(be, bits, d, g, T):
    """The reference-shaped entry (CudaQuantAttnArgs): packed + residual, host score read-back."""
    hkv = 2
    case = pack_with_oracle(wl.kivi_source(1000 + bits + T, [T], hkv * g, hkv, d, 128, bits))
    want, want_p = _oracle_kivi(case, 0, scores=True)
    out = torch.full((case.hq, d), float("nan"), device="cuda")
    stride = T + 5
    sc = torch.full((case.hq, stride), -1.0)
    qk = _dev(case.qk[0]) if case.qk[0].size else None
    qv = _dev(case.qv[0]) if case.qv[0].size else None
    rc = be.attention_gen_quant(_dev(case.q[0]), qk, qv, _dev(case.res_k[0]), _dev(case.res_v[0]), out, case.hq, hkv, d,
                                case.q_tokens[0], case.res_tokens[0], 128, 1.0 / np.sqrt(d), bits, scores_out=sc)
    assert rc == 0
    np.testing.assert_allclose(out.cpu().numpy(), want, atol=OUT_ATOL, rtol=OUT_RTOL)
    np.testing.assert_allclose(sc.numpy()[:, :T], want_p, atol=P_ATOL, rtol=P_RTOL)
    assert be.check_status() == 0


def test_residual_only_matches_f64(be):
    """Case A of the reference's device harness (engine/src/bin/test_cuda_quant_attn_device.rs:108-200):
    no packed tokens, residual ring only, against a host F64 reference at 1e-4."""
    hq, hkv, d, rt = 8, 2, 64, 20
    rng = np.random.default_rng(3)
    q = rng.standard_normal((hq, d)).astype(np.float32)
    rk = np.zeros((hkv, 128, d), dtype=np.float32)
    rv = np.zeros_like(rk)
    rk[:, :rt] = rng.standard_normal((hkv, rt, d))
    rv[:, :rt] = rng.standard_normal((hkv, rt, d))
    out = torch.zeros(hq, d, device="cuda")
    scale = 0.37   # an arbitrary scale: the entry takes it from the caller
    assert be.attention_gen_quant(_dev(q), None, None, _dev(rk), _dev(rv), out, hq, hkv, d, 0, rt, 128, scale, 4) == 0
    want = np.zeros((hq, d))
    for h in range(hq):
        s = rk[h // 4, :rt].astype(np.float64) @ q[h].astype(np.float64) * scale
        p = np.exp(s - s.max())
        want[h] = (p / p.sum()) @ rv[h // 4, :rt].astype(np.float64)
    np.testing.assert_allclose(out.cpu().numpy(), want, atol=1e-4)


def test_exactly_representable_q2_blocks(be):
    """Case B of the same harness: Q2 blocks whose values are exact (codes 0..3, d=1, m=0)."""
    hq, hkv, d = 4, 1, 64
    T = 128
    k = (np.arange(T * d).reshape(T, 1, d) % 4).astype(np.float32)
    v = ((np.arange(T * d).reshape(T, 1, d) // 3) % 4).astype(np.float32)
    c = orc.KiviCache(hkv, d, 128, 2)
    c.update(k, v)
    c.update(k[:1], v[:1])
    qk, qv, rk, rv = c.export()
    q = orc.lcg(hq * d, 5).reshape(hq, d) * 0.1
    out = torch.zeros(hq, d, device="cuda")
    assert be.attention_gen_quant(_dev(q), _dev(qk), _dev(qv), _dev(rk), _dev(rv), out, hq, hkv, d, 128, 1, 128,
                                  1 / 8.0, 2) == 0
    kk = np.concatenate([k, k[:1]])[:, 0].astype(np.float64)
    vv = np.concatenate([v, v[:1]])[:, 0].astype(np.float64)
    s = kk @ q.astype(np.float64).T / 8.0
    p = np.exp(s - s.max(0))
    want = (p / p.sum(0)).T @ vv
    np.testing.assert_allclose(out.cpu().numpy(), want, atol=1e-3)


@pytest.mark.parametrize("g", [1, 4, 8])
@pytest.mark.parametrize("T", [128 * 2 + 1, 128 * 7 + 100, 128 * 70 + 5, 128 * 301])
def test_q4_d128_lengths_and_groups(be, g, T):
    """Q4 at head_dim 128 (the benchmarked format): ragged last group, several splits at the longer lengths, GQA 1/4/8,
    against the oracle, with scores."""
    hkv, d = 2, 128
    case = pack_with_oracle(wl.kivi_source(77 + T + g, [T], hkv * g, hkv, d, 128, 4))
    want, want_p = _oracle_kivi(case, 0, scores=True)
    out = torch.full((case.hq, d), float("nan"), device="cuda")
    sc = torch.full((case.hq, T), -1.0)
    rc = be.attention_gen_quant(_dev(case.q[0]), _dev(case.qk[0]), _dev(case.qv[0]), _dev(case.res_k[0]),
                                _dev(case.res_v[0]), out, case.hq, hkv, d, case.q_tokens[0], case.res_tokens[0], 128,
                                1.0 / np.sqrt(d), 4, scores_out=sc)
    assert rc == 0
    np.testing.assert_allclose(out.cpu().numpy(), want, atol=OUT_ATOL, rtol=OUT_RTOL)
    np.testing.assert_allclose(sc.numpy(), want_p, atol=P_ATOL, rtol=P_RTOL)
    assert be.check_status() == 0


@pytest.mark.parametrize("res_f16", [False, True])
def test_batched_kivi_q4_h2o_reduced(be, res_f16):
    """The benchmarked KIVI workload scaled down (B=3, T in {4224, 2048+128, 777}): Q4, 1% of K channels x8, fused H2O
    group-mean vector [B,Hkv,T] and flat sums; F32 ring (engine) and F16 residual (benchmark wording)."""
    from argus_engine_b200 import DecodeExtras


    lens = [4224, 2176, 777]
    case = pack_with_oracle(wl.kivi_source(2, lens, 32, 8, 128, 128, 4), res_f16=res_f16)
    B, stride = len(lens), 4352
    seqs = [(_dev(case.qk[i]), _dev(case.qv[i]), _dev(case.res_k[i]), _dev(case.res_v[i]), case.q_tokens[i],
             case.res_tokens[i]) for i in range(B)]
    out = torch.full((B, 32, 128), float("nan"), device="cuda")
    ex = DecodeExtras(head_scores=torch.zeros(B, 8, stride, device="cuda"), flat_scores=torch.zeros(B, stride, device="cuda"),
                      score_stride=stride)
    be.kivi_attention_batched(_dev(case.q), seqs, out, 32, 8, 128, 128, 4, 1 / np.sqrt(128), res_f16=res_f16, extras=ex)
    torch.cuda.synchronize()
    assert be.check_status() == 0
    for i, T in enumerate(lens):
        want, want_p = _oracle_kivi(case, i, scores=True)
        np.testing.assert_allclose(out[i].cpu().numpy(), want, atol=OUT_ATOL, rtol=OUT_RTOL)
        sf = np.zeros(stride, dtype=np.float32)
        sh = np.zeros(8 * stride, dtype=np.float32)
        orc.score_accumulate_layer(want_p, T, 32, 8, stride, sf, sh)
        np.testing.assert_allclose(ex.head_scores[i].cpu().numpy()[:, :T], sh.reshape(8, stride)[:, :T], atol=P_ATOL,
                                   rtol=P_RTOL)
        np.testing.assert_allclose(ex.flat_scores[i].cpu().numpy()[:T], sf[:T], atol=P_ATOL, rtol=P_RTOL)
        # eviction index selection on these scores is identical (heavy hitters are well separated here)
        got_keep = orc.h2o_keep(T, 4, 64, 128, ex.flat_scores[i].cpu().numpy()[:T])
        assert got_keep == orc.h2o_keep(T, 4, 64, 128, sf[:T])


@pytest.mark.parametrize("bits", [2, 4, 8])
@pytest.mark.parametrize("d,g", [(128, 4), (64, 8)])
def test_degenerate_blocks_through_the_folded_scales(be, bits, d, g):
    """Blocks whose scale or minimum is special - constant channels and tokens (d == 0), all-zero blocks, a range that
    underflows F16 (d stored as 0), large offsets with a small range (|m| >> d), a strongly scaled query - go through
    q*d / p*d and the bias MMAs like any other block and still match the oracle."""
    hkv, T = 2, 128 * 3 + 40
    src = wl.kivi_source(77 + bits, [T], hkv * g, hkv, d, 128, bits)
    k, v = src.k[0], src.v[0]
    rng = np.random.default_rng(3)
    k[:, 0, 0] = 3.25                                   # constant K channel: every block has d == 0
    k[:, 0, 1] = 0.0                                    # all-zero channel
    k[:, 0, 2] = rng.standard_normal(T) * 1e-30         # range far below the smallest F16 scale
    k[:, 0, 3] = 100.0 + rng.standard_normal(T) * 0.01  # |m| >> d
    k[:, 1, 5] = -50.0 + rng.standard_normal(T)
    v[7, :, :] = 1.0                                    # constant V token
    v[8, :, :] = 0.0
    v[:, 1, 32:64] = 200.0 + rng.standard_normal((T, 32)).astype(np.float32) * 0.05
    v[9, 0, :32] = np.arange(32) * 0.5                  # .5 ties along a V block
    src.q[0] *= 4.0
    case = pack_with_oracle(src)
    want, want_p = _oracle_kivi(case, 0, scores=True)
    out = torch.full((case.hq, d), float("nan"), device="cuda")
    sc = torch.full((case.hq, T), -1.0)
    rc = be.attention_gen_quant(_dev(case.q[0]), _dev(case.qk[0]), _dev(case.qv[0]), _dev(case.res_k[0]), _dev(case.res_v[0]),
                                out, case.hq, hkv, d, case.q_tokens[0], case.res_tokens[0], 128, 1.0 / np.sqrt(d), bits,
                                scores_out=sc)
    assert rc == 0 and be.check_status() == 0
    np.testing.assert_allclose(out.cpu().numpy(), want, atol=OUT_ATOL, rtol=OUT_RTOL)
    np.testing.assert_allclose(sc.numpy(), want_p, atol=P_ATOL, rtol=P_RTOL)


@pytest.mark.parametrize("bits", [2, 4, 8])
def test_paged_kivi_matches_contiguous_and_oracle(be, bits):
    """Flushes of three sequences scattered over one page pool (a page = one flush of all KV heads, in shuffled order
    with unused pages between): outputs and score vectors are bit-identical to the contiguous call, which is checked
    against the oracle."""
    from argus_engine_b200 import DecodeExtras

    hq, hkv, d, rc = 32, 8, 128, 128
    lens = [128 * 9 + 50, 128 * 4, 77]
    case = pack_with_oracle(wl.kivi_source(11, lens, hq, hkv, d, rc, bits))
    B, stride = len(lens), 128 * 10
    bb = {2: 12, 4: 20, 8: 36}[bits]
    kpage = hkv * (rc // 32) * d * bb
    vpage = hkv * rc * (d // 32) * bb
    flushes = [case.q_tokens[i] // rc for i in range(B)]
    n_pages = sum(flushes) + 5
    rng = np.random.default_rng(5)
    order = rng.permutation(n_pages)[:sum(flushes)].astype(np.int32)
    qk_pool = rng.integers(0, 256, n_pages * kpage, dtype=np.uint8)     # unused pages hold garbage
    qv_pool = rng.integers(0, 256, n_pages * vpage, dtype=np.uint8)
    tables, at = [], 0
    for i in range(B):
        t = order[at:at + flushes[i]]
        at += flushes[i]
        kb = np.asarray(case.qk[i]).view(np.uint8).reshape(-1)
        vb = np.asarray(case.qv[i]).view(np.uint8).reshape(-1)
        for f, page in enumerate(t):
            qk_pool[page * kpage:(page + 1) * kpage] = kb[f * kpage:(f + 1) * kpage]
            qv_pool[page * vpage:(page + 1) * vpage] = vb[f * vpage:(f + 1) * vpage]
        tables.append(_dev(t) if len(t) else None)
    scale = 1 / np.sqrt(d)

    def extras():
        return DecodeExtras(head_scores=torch.zeros(B, hkv, stride, device="cuda"),
                            flat_scores=torch.zeros(B, stride, device="cuda"), score_stride=stride)

    seqs = [(_dev(case.qk[i]), _dev(case.qv[i]), _dev(case.res_k[i]), _dev(case.res_v[i]), case.q_tokens[i],
             case.res_tokens[i]) for i in range(B)]
    out_c = torch.full((B, hq, d), float("nan"), device="cuda")
    ex_c = extras()
    be.kivi_attention_batched(_dev(case.q), seqs, out_c, hq, hkv, d, rc, bits, scale, extras=ex_c)
    pseqs = [(tables[i], _dev(case.res_k[i]), _dev(case.res_v[i]), case.q_tokens[i], case.res_tokens[i]) for i in range(B)]
    out_p = torch.full((B, hq, d), float("nan"), device="cuda")
    ex_p = extras()
    be.kivi_attention_paged(_dev(case.q), _dev(qk_pool), _dev(qv_pool), pseqs, out_p, hq, hkv, d, rc, bits, scale,
                            extras=ex_p)
    torch.cuda.synchronize()
    assert be.check_status() == 0
    assert torch.equal(out_p, out_c)
    assert torch.equal(ex_p.head_scores, ex_c.head_scores) and torch.equal(ex_p.flat_scores, ex_c.flat_scores)
    for i in range(B):
        np.testing.assert_allclose(out_p[i].cpu().numpy(), _oracle_kivi(case, i, scores=True)[0], atol=OUT_ATOL, rtol=OUT_RTOL)
    # a sequence with packed tokens and no page table is refused
    from argus_engine_b200 import ArgusB200Error
    with pytest.raises(ArgusB200Error):
        be.kivi_attention_paged(_dev(case.q), _dev(qk_pool), _dev(qv_pool), [(None,) + pseqs[0][1:]] + pseqs[1:], out_p,
                                hq, hkv, d, rc, bits, scale)


@pytest.mark.parametrize("case_id", [0, 1])
def test_score_reduce_vs_oracle(be, case_id):
    """CudaScoreReduceBackend: the hand-computed case of engine/src/bin/test_cuda_gpu_score_device.rs:36-118
    and a random multi-layer case, bit-identical to the restated reference kernel."""
    if case_id == 0:
        L, hq, hkv, max_seq, T = 2, 2, 1, 8, 3
        s = np.zeros((L, hq, max_seq), dtype=np.float32)
        s[0, 0, :3], s[0, 1, :3] = [0.1, 0.2, 0.7], [0.3, 0.3, 0.4]
        s[1, 0, :3], s[1, 1, :3] = [0.5, 0.4, 0.1], [0.2, 0.2, 0.6]
    else:
        L, hq, hkv, max_seq, T = 5, 32, 8, 700, 611
        s = np.random.default_rng(0).random((L, hq, max_seq), dtype=np.float32)
    sd = _dev(s)
    imp = torch.zeros(max_seq, device="cuda")
    himp = torch.zeros(hkv * max_seq, device="cuda")
    lflat = torch.zeros(L * max_seq, device="cuda")
    w_imp, w_himp, w_lf = np.zeros(max_seq, np.float32), np.zeros(hkv * max_seq, np.float32), np.zeros(L * max_seq, np.float32)
    for decay in (1.0, 0.5, 0.9):   # 0.9: importance*decay is inexact, so the rounding order (multiply, then add) shows
        if decay == 0.9 and case_id == 0:
            np.testing.assert_allclose(w_imp[:3], 1.5 * np.array([0.7, 0.6, 1.1]), atol=1e-5)   # the hand-computed case
        assert be.score_reduce(sd, imp, himp, decay, L, hq, hkv, T, max_seq, max_seq) == 0
        assert be.score_reduce_per_layer(sd, lflat, decay, L, hq, hkv, T, max_seq, max_seq) == 0
        orc.score_fused_reduce(s, w_imp, w_himp, decay, L, hq, hkv, T, max_seq, max_seq)
        orc.score_reduce_per_layer(s, w_lf, decay, L, hq, T, max_seq, max_seq)
    torch.cuda.synchronize()
    assert np.array_equal(imp.cpu().numpy(), w_imp)
    assert np.array_equal(himp.cpu().numpy(), w_himp)
    assert np.array_equal(lflat.cpu().numpy(), w_lf)


@pytest.mark.parametrize("bits", [2, 4, 8])
def test_device_cache_matches_oracle_container(be, bits):
    """The device-resident container (ring write + device flush) ends up with exactly the bytes of the
    restated engine container, for prompt-sized and token-by-token updates, and decodes to the same result."""
    from argus_engine_b200.kivi_cache import KiviDeviceCache

    hkv, d, rc, T = 2, 64, 64, 64 * 3 + 21
    src = wl.kivi_source(77 + bits, [T], 8, hkv, d, rc, bits)
    want = pack_with_oracle(src)
    cache = KiviDeviceCache(be, hkv, d, 1024, rc, bits)
    k, v = _dev(src.k[0]), _dev(src.v[0])
    cache.update(k[:150], v[:150])            # a prefill-sized write crossing two flushes
    for t in range(150, T):                   # then token by token
        cache.update(k[t:t + 1], v[t:t + 1])
    torch.cuda.synchronize()
    assert (cache.q_tokens, cache.res_pos) == (want.q_tokens[0], want.res_tokens[0])
    assert np.array_equal(cache.qk.cpu().numpy()[:want.qk[0].size], want.qk[0])
    assert np.array_equal(cache.qv.cpu().numpy()[:want.qv[0].size], want.qv[0])
    assert np.array_equal(cache.res_k.cpu().numpy()[:, :cache.res_pos], want.res_k[0][:, :cache.res_pos])
    out = torch.zeros(1, 8, d, device="cuda")
    be.kivi_attention_batched(_dev(src.q), [cache.seq()], out, 8, hkv, d, rc, bits, 1 / np.sqrt(d))
    torch.cuda.synchronize()
    ref, _ = _oracle_kivi(want, 0)
    np.testing.assert_allclose(out[0].cpu().numpy(), ref, atol=OUT_ATOL, rtol=OUT_RTOL)
