"""Pins the CPU oracle against the known-answer tests the reference keeps for this path.

Each case re-states a reference unit test (file:line given) using only its formulas and literals.
"""
import numpy as np
import pytest

from oracle import oracle as orc


def _block(d, m, qs):
    hdr = np.array([d, m], dtype=np.float16).view(np.uint8)
    return np.concatenate([hdr, np.asarray(qs, dtype=np.uint8)])


# crates/argus-kv-codec/src/lib.rs:32,121,171,457 — on-device block sizes
def test_block_sizes():
    assert (orc.block_bytes(2), orc.block_bytes(4), orc.block_bytes(8)) == (12, 20, 36)


# crates/argus-kv-codec/src/lib.rs:303-319
def test_q2_dequantize_known():
    out = orc.kv_dequantize(_block(2.0, -1.0, [0b11100100] * 8), 2)
    np.testing.assert_allclose(out, np.tile([-1.0, 1.0, 3.0, 5.0], 8), atol=0.01)


# crates/argus-kv-codec/src/lib.rs:382-394
def test_q4_known_values():
    out = orc.kv_dequantize(_block(1.0, -2.0, [0x31] * 16), 4)
    np.testing.assert_allclose(out, np.tile([-1.0, 1.0], 16), atol=0.01)


# crates/argus-kv-codec/src/lib.rs:212-300,352-453 — zeros, constants, round-trip error bounds
@pytest.mark.parametrize("bits,levels", [(2, 3), (4, 15), (8, 255)])
def test_codec_bounds(bits, levels):
    z = orc.kv_dequantize(orc.kv_quantize(np.zeros(32), bits), bits)
    assert np.all(z == 0.0)
    c = orc.kv_dequantize(orc.kv_quantize(np.full(32, 42.0), bits), bits)
    assert np.all(np.abs(c - 42.0) < 0.1)
    src = np.arange(32, dtype=np.float32) * 0.1
    rt = orc.kv_dequantize(orc.kv_quantize(src, bits), bits)
    assert np.max(np.abs(rt - src)) < 3.1 / (2 * levels) + 0.02
    neg = (-10.0 + np.arange(32) * 9.0 / 31.0).astype(np.float32)
    rt = orc.kv_dequantize(orc.kv_quantize(neg, bits), bits)
    assert np.max(np.abs(rt - neg)) < 9.0 / (2 * levels) + 0.05


# crates/argus-kv-codec/src/lib.rs:283-300 — exact 0..3 values pack LSB-first, 4 codes per byte
def test_q2_manual_pack_bits():
    src = (np.arange(32) % 4).astype(np.float32)
    blk = orc.kv_quantize(src, 2)
    assert blk[4:].tolist() == [0b11100100] * 8
    assert np.frombuffer(blk[:4].tobytes(), dtype=np.float16).tolist() == [1.0, 0.0]


def test_q4_pack_nibble_order_and_rounding():
    # codes are computed with the un-rounded F32 scale; .5 ties round away from zero
    src = np.zeros(32, dtype=np.float32)
    src[1] = 15.0
    src[2] = 0.5   # (0.5 - 0) * 1 = 0.5 -> 1
    src[3] = 2.5   # -> 3
    blk = orc.kv_quantize(src, 4)
    assert blk[4] == (0 | (15 << 4))
    assert blk[5] == (1 | (3 << 4))


# engine/src/kv/quant_window_cache.rs:2761-2850 — flush happens at the write AFTER the ring fills,
# residual rows are the exact F32 inputs
def test_kivi_flush_timing_and_residual_exact():
    hkv, d, rc = 2, 32, 32
    rng = np.random.default_rng(0)
    c = orc.KiviCache(hkv, d, rc, 4)
    k = rng.standard_normal((rc + 1, hkv, d)).astype(np.float32)
    v = rng.standard_normal((rc + 1, hkv, d)).astype(np.float32)
    c.update(k[:rc], v[:rc])
    assert (c.q_tokens, c.res_tokens) == (0, rc)
    c.update(k[rc:], v[rc:])
    assert (c.q_tokens, c.res_tokens) == (rc, 1)
    qk, qv, rk, rv = c.export()
    assert qk.size == hkv * (rc // 32) * d * 20 and qv.size == hkv * rc * (d // 32) * 20
    np.testing.assert_array_equal(rk[:, 0, :], k[rc])
    np.testing.assert_array_equal(rv[:, 0, :], v[rc])
    # block order: K blocks [h][group][ch] hold 32 tokens of one channel; V blocks [h][tok][blk]
    kb = orc.kv_dequantize(qk, 4).reshape(hkv, rc // 32, d, 32)
    ref = orc.kv_dequantize(orc.kv_quantize(np.ascontiguousarray(k[:rc, 1, 5]), 4), 4)
    np.testing.assert_array_equal(kb[1, 0, 5], ref)
    vb = orc.kv_dequantize(qv, 4).reshape(hkv, rc, d)
    ref = orc.kv_dequantize(orc.kv_quantize(v[7, 0], 4), 4)
    np.testing.assert_array_equal(vb[0, 7], ref)


# engine/src/kv/quant_window_cache.rs:3285-3322 — Q4 view error bound; view is SeqMajor [T,Hkv,D]
def test_kivi_view_error_bound():
    hkv, d, rc, T = 2, 64, 64, 150
    rng = np.random.default_rng(1)
    k = rng.standard_normal((T, hkv, d)).astype(np.float32)
    v = rng.standard_normal((T, hkv, d)).astype(np.float32)
    c = orc.KiviCache(hkv, d, rc, 4)
    for t in range(T):
        c.update(k[t:t + 1], v[t:t + 1])
    assert (c.q_tokens, c.res_tokens) == (128, 22)
    qk, qv, rk, rv = c.export()
    vk, vv = orc.kivi_assemble_view(qk, qv, rk, rv, hkv, d, rc, 4, c.q_tokens, c.res_tokens)
    np.testing.assert_array_equal(vk[128:], k[128:])
    np.testing.assert_array_equal(vv[128:], v[128:])
    assert np.max(np.abs(vk[:128] - k[:128])) < 8.0 / 30 + 0.05
    assert np.max(np.abs(vv[:128] - v[:128])) < 8.0 / 30 + 0.05


# engine/src/bin/test_cuda_gpu_score_device.rs:36-118 — hand-computed MAX / GQA mean / decay
def test_score_reduce_hand_computed():
    L, hq, hkv, max_seq, T = 2, 2, 1, 8, 3
    s = np.zeros((L, hq, max_seq), dtype=np.float32)
    s[0, 0, :3] = [0.1, 0.2, 0.7]
    s[0, 1, :3] = [0.3, 0.3, 0.4]
    s[1, 0, :3] = [0.5, 0.4, 0.1]
    s[1, 1, :3] = [0.2, 0.2, 0.6]
    imp = np.zeros(max_seq, dtype=np.float32)
    himp = np.zeros(hkv * max_seq, dtype=np.float32)
    orc.score_fused_reduce(s, imp, himp, 1.0, L, hq, hkv, T, max_seq, max_seq)
    np.testing.assert_allclose(imp[:3], [0.7, 0.6, 1.1], atol=1e-5)
    np.testing.assert_allclose(himp[:3], [0.35, 0.30, 0.55], atol=1e-5)
    imp[:] = 0
    himp[:] = 0
    for _ in range(2):
        orc.score_fused_reduce(s, imp, himp, 0.5, L, hq, hkv, T, max_seq, max_seq)
    np.testing.assert_allclose(imp[:3], 1.5 * np.array([0.7, 0.6, 1.1]), atol=1e-5)
    # CPU producer path (attn-score/src/lib.rs:244-359): same numbers through begin/accumulate/end
    imp[:] = 0
    himp[:] = 0
    sf = np.zeros(max_seq, dtype=np.float32)
    sh = np.zeros(hkv * max_seq, dtype=np.float32)
    orc.score_begin_step(imp, himp, sf, sh, hkv, max_seq, 0.0)
    for l in range(L):
        orc.score_accumulate_layer(s[l], T, hq, hkv, max_seq, sf, sh)
    orc.score_end_step(imp, himp, sf, sh, hkv, max_seq)
    np.testing.assert_allclose(imp[:3], [0.7, 0.6, 1.1], atol=1e-5)
    np.testing.assert_allclose(himp[:3], [0.35, 0.30, 0.55], atol=1e-5)
    lf = np.zeros(L * max_seq, dtype=np.float32)
    orc.score_reduce_per_layer(s, lf, 1.0, L, hq, T, max_seq, max_seq)
    np.testing.assert_allclose(lf.reshape(L, max_seq)[:, :3], [[0.4, 0.5, 1.1], [0.7, 0.6, 0.7]], atol=1e-5)


# crates/argus-extension-api/src/lib.rs:3136-3200 — keep-list literals
def test_keep_top_k_literals():
    sc = np.zeros(20, dtype=np.float32)
    sc[[6, 9, 12, 14]] = [10, 9, 8, 7]
    assert orc.keep_top_k(20, 4, 4, 4, sc) == [0, 1, 2, 3, 6, 9, 12, 14, 16, 17, 18, 19]
    assert orc.keep_top_k(20, 4, 6, 0, None) == [0, 1, 2, 3, 14, 15, 16, 17, 18, 19]
    tie = np.zeros(8, dtype=np.float32)
    tie[[3, 4]] = 5.0
    assert orc.keep_top_k(8, 2, 2, 1, tie) == [0, 1, 3, 6, 7]
    assert orc.keep_top_k(2, 4, 4, 0, None) == [0, 1]


# crates/techniques/h2o/src/lib.rs:429-482
def test_h2o_keep_lists():
    assert orc.h2o_keep(10, 0, 4, 6) is None
    assert orc.h2o_keep(20, 0, 4, 6) == list(range(10, 20))
    imp = np.zeros(20, dtype=np.float32)
    imp[5], imp[9], imp[2] = 10.0, 9.0, 1.0
    assert orc.h2o_keep(20, 0, 2, 4, imp) == [5, 9, 16, 17, 18, 19]


def _naive_decode(q, k, v, hq, hkv, d, T):
    """F64 three-pass reference on HeadMajor [Hkv,cap,D] float arrays."""
    g = hq // hkv
    out = np.zeros((hq, d))
    p_all = np.zeros((hq, T))
    for h in range(hq):
        s = (k[h // g, :T].astype(np.float64) @ q[h].astype(np.float64)) / np.sqrt(d)
        p = np.exp(s - s.max())
        p /= p.sum()
        p_all[h] = p
        out[h] = p @ v[h // g, :T].astype(np.float64)
    return out, p_all


# engine/src/backend/cpu/x86.rs:1811-1973 — AVX2 arm vs scalar arm on LCG data, tol 1e-4 (F32) / 1e-3 (F16),
# both layouts; engine/tests/test_attention_flash_decoding.rs:260-376 — chunk-boundary lengths
@pytest.mark.parametrize("T", [1, 31, 33, 1023, 1025, 2500])
@pytest.mark.parametrize("head_major", [True, False])
def test_decode_avx2_vs_scalar_vs_f64(T, head_major):
    hq, hkv, d = 8, 2, 64
    q = orc.lcg(hq * d, 42).reshape(hq, d)
    kf = orc.lcg(hkv * T * d, 123).reshape(hkv, T, d)
    vf = orc.lcg(hkv * T * d, 456).reshape(hkv, T, d)
    k16, v16 = orc.f32_to_f16_bits(kf), orc.f32_to_f16_bits(vf)
    kr, vr = k16.view(np.float16).astype(np.float32), v16.view(np.float16).astype(np.float32)
    want, want_p = _naive_decode(q, kr, vr, hq, hkv, d, T)
    if not head_major:
        k16, v16 = (np.ascontiguousarray(a.transpose(1, 0, 2)) for a in (k16, v16))
    o1, s1 = orc.attention_gen(q, k16, v16, hq, hkv, d, T, head_major, want_scores=True)
    o2, s2 = orc.attention_gen(q, k16, v16, hq, hkv, d, T, head_major, want_scores=True, avx2=True)
    np.testing.assert_allclose(o1, want, atol=1e-4)
    np.testing.assert_allclose(o2, o1, atol=1e-3)
    np.testing.assert_allclose(s1, want_p, atol=1e-5)
    np.testing.assert_allclose(s2, s1, atol=1e-5)
    np.testing.assert_allclose(s1.sum(axis=1), 1.0, atol=1e-4)


def test_decode_single_token_and_uniform():
    hq, hkv, d = 4, 2, 32
    q = orc.lcg(hq * d, 1).reshape(hq, d)
    v = orc.lcg(hkv * 5 * d, 2).reshape(hkv, 5, d)
    o, _ = orc.attention_gen(q, v.copy(), v, hq, hkv, d, 1)
    np.testing.assert_allclose(o, v[[0, 0, 1, 1], 0], atol=1e-6)  # T=1 -> out = V row
    o, s = orc.attention_gen(q, np.zeros_like(v), v, hq, hkv, d, 5, want_scores=True)  # K=0 -> uniform
    np.testing.assert_allclose(s, 0.2, atol=1e-6)
    np.testing.assert_allclose(o, v.mean(axis=1)[[0, 0, 1, 1]], atol=1e-5)
    # NaN guard of the CPU backends (engine/src/backend/cpu/common.rs:555-584)
    kn = np.full_like(v, np.nan)
    o, s = orc.attention_gen(q, kn, v, hq, hkv, d, 5, want_scores=True, guards=True)
    np.testing.assert_allclose(s, 0.2, atol=1e-6)


def _naive_prefill(q, k, v, hq, hkv, S, T, d):
    B = q.shape[0]
    g = hq // hkv
    out = np.zeros_like(q, dtype=np.float64)
    for b in range(B):
        for h in range(hq):
            s = q[b, :, h].astype(np.float64) @ k[b, h // g, :T].astype(np.float64).T / np.sqrt(d)
            mask = np.arange(T)[None, :] <= (np.arange(S)[:, None] + T - S)
            s = np.where(mask, s, -np.inf)
            p = np.exp(s - s.max(axis=1, keepdims=True))
            p /= p.sum(axis=1, keepdims=True)
            out[b, :, h] = p @ v[b, h // g, :T].astype(np.float64)
    return out


# engine/tests/test_prefill_flash_attention.rs (GQA 1/2/4/8, ragged tiles, continuation) and
# engine/src/backend/cuda_pc.rs:2272-2577 (single token => V; cache_seq_len > seq_len)
@pytest.mark.parametrize("S,T,g", [(1, 1, 1), (33, 33, 2), (70, 70, 4), (16, 50, 8), (64, 64, 1)])
def test_prefill_vs_naive(S, T, g):
    B, hkv, d, cap = 2, 2, 32, 80
    hq = hkv * g
    q = orc.lcg(B * S * hq * d, 7).reshape(B, S, hq, d)
    k = orc.lcg(B * hkv * cap * d, 8).reshape(B, hkv, cap, d)
    v = orc.lcg(B * hkv * cap * d, 9).reshape(B, hkv, cap, d)
    got = orc.flash_prefill(q, k, v, hq, hkv, S, T, d, cap)
    np.testing.assert_allclose(got, _naive_prefill(q, k, v, hq, hkv, S, T, d), atol=1e-4)
    if S == 1 and T == 1:
        np.testing.assert_allclose(got[:, 0], v[:, :, 0].repeat(g, axis=1), atol=1e-6)
    ks, vs = (np.ascontiguousarray(a.transpose(0, 2, 1, 3)) for a in (k, v))
    got_s = orc.flash_prefill(q, ks, vs, hq, hkv, S, T, d, cap, head_major=False)
    np.testing.assert_array_equal(got_s, got)


# engine/src/kv/quant_window_format.rs:524-586 and standard_format.rs:3141 — K = 0 => row r = mean(V[0..=r])
def test_prefill_causal_uniform():
    B, hq, hkv, S, d = 1, 2, 1, 40, 32
    q = orc.lcg(S * hq * d, 3).reshape(B, S, hq, d)
    v = orc.lcg(S * d, 4).reshape(B, hkv, S, d)
    got = orc.flash_prefill(q, np.zeros_like(v), v, hq, hkv, S, S, d, S)
    want = np.cumsum(v[0, 0].astype(np.float64), axis=0) / np.arange(1, S + 1)[:, None]
    np.testing.assert_allclose(got[0, :, 0], want, atol=1e-5)
    np.testing.assert_allclose(got[0, :, 1], want, atol=1e-5)


# engine/src/backend/cpu/neon.rs:1044-1125 — merged split partials equal the unsplit result
def test_lse_merge_equals_unsplit():
    hq, hkv, d, T = 4, 1, 32, 1000
    q = orc.lcg(hq * d, 11).reshape(hq, d)
    k = orc.lcg(T * d, 12).reshape(1, T, d)
    v = orc.lcg(T * d, 13).reshape(1, T, d)
    full, _ = orc.attention_gen(q, k, v, hq, hkv, d, T)
    cuts = [0, 1, 257, 700, 1000]
    for h in range(hq):
        os_, ls = [], []
        for a, b in zip(cuts[:-1], cuts[1:]):
            s = (k[0, a:b] @ q[h]) / np.sqrt(d)
            m = s.max()
            e = np.exp(s - m)
            os_.append((e / e.sum()) @ v[0, a:b])
            ls.append(m + np.log(e.sum()))
        os_.append(np.zeros(d))
        ls.append(-np.inf)  # an empty shard is skipped
        np.testing.assert_allclose(orc.lse_merge(np.array(os_), np.array(ls)), full[h], atol=1e-5)


# ── KV executors: the numpy restatements against hand-worked cases ──

def test_compact_keep_positions_hand_case():
    """keep = [0, 1, 5, 6, 9] at write_start 0 (engine/src/kv/kv_cache.rs:1266-1300): the run (0,1) stays, (5,6) moves
    to 2..3, 9 moves to 4; everything behind position 4 keeps its old contents."""
    cache = np.arange(2 * 12 * 4, dtype=np.float32).reshape(2, 12, 4)
    want = cache.copy()
    want[:, 2] = cache[:, 5]
    want[:, 3] = cache[:, 6]
    want[:, 4] = cache[:, 9]
    orc.compact_keep_positions(cache, [0, 1, 5, 6, 9], 0)
    assert np.array_equal(cache, want)
    one = np.arange(2 * 12 * 4, dtype=np.float32).reshape(2, 12, 4)
    ref = one.copy()
    orc.compact_keep_positions(one, [3, 4], 1, head=1)   # per-head variant, write_start 1
    ref[1, 1], ref[1, 2] = ref[1, 3].copy(), ref[1, 4].copy()
    assert np.array_equal(one, ref)


def test_apply_weighted_merges_hand_case():
    """acc = into_w*into + w1*from1 + w2*from2 with every step rounded to F32 (standard_format.rs:860-875), F16 rounds once
    at the store (:878-893)."""
    k = np.zeros((1, 4, 2), dtype=np.float32)
    k[0, 0], k[0, 1], k[0, 2] = [1.0, 2.0], [10.0, 20.0], [100.0, 200.0]
    v = k.copy()
    orc.apply_weighted_merges(k, v, [(0, np.float32(0.5), [(1, np.float32(0.25)), (2, np.float32(0.125))])], axis=1)
    assert np.array_equal(k[0, 0], np.float32([0.5 + 2.5 + 12.5, 1.0 + 5.0 + 25.0]))
    assert np.array_equal(v[0, 0], np.float32([1.0, 2.0]))   # key-only merge leaves V alone
    h = np.float16([[[0.1, 0.2], [0.3, 0.4]]])
    hv = h.copy()
    orc.apply_weighted_merges(h, hv, [(0, np.float32(0.7), [(1, np.float32(0.3))])])
    a = np.float32(0.7) * np.float16([0.1, 0.2]).astype(np.float32)
    a = a + np.float32(0.3) * np.float16([0.3, 0.4]).astype(np.float32)
    assert np.array_equal(h[0, 0], a.astype(np.float16))


def test_kv_scatter_rounds_to_nearest_even():
    src = np.float32([[[1.0 + 2 ** -11, 1.0 + 3 * 2 ** -11, 65520.0, 1e-8]]])   # ties to even: 1.0 and 1.00195; inf; 0
    k = np.zeros((1, 2, 4), dtype=np.float16)
    v = np.zeros_like(k)
    orc.kv_scatter(src, src, k, v, 1)
    assert k[0, 1].tolist() == [1.0, float(np.float16(1.0 + 2 ** -9)), float("inf"), 0.0]
    assert not k[0, 0].any()


def test_prefill_attention_scores_on_the_reference_test_inputs():
    """Inputs of pfa_bit_exact_matches_eager_reference (engine/src/kv/standard_format.rs:3397-3460): q[i] = ((i % 13) - 6)*0.1,
    k[i] = ((i % 17) - 8)*0.07, head_dim 8, seq_len 6, q_window 3, HeadMajor capacity 16, GQA 4:2, with and without a
    sliding window of 4. Each window row is a distribution over its visible keys, so every head's summed seed has mass
    q_window, keys outside a row's band get nothing, and the per-row outputs add up to the summed one bit for bit."""
    nq, nkv, d, S, cap, qw = 4, 2, 8, 6, 16, 3
    q = np.array([((i % 13) - 6.0) * 0.1 for i in range(S * nq * d)], dtype=np.float32).reshape(S, nq, d)
    k = np.array([((i % 17) - 8.0) * 0.07 for i in range(nkv * cap * d)], dtype=np.float32).reshape(nkv, cap, d)
    for window in (None, 4):
        s, rows, mean = orc.prefill_attention_scores(q, k, nkv, 0, qw, S, window)
        assert np.allclose(s.sum(1), qw, atol=1e-5)
        acc = np.zeros_like(s)
        for r in range(qw):
            acc += rows[r]
        assert np.array_equal(acc, s)
        for step, r in enumerate(range(S - qw, S)):
            lo = 0 if window is None else max(0, r - 3)
            assert not rows[step, :, :lo].any() and not rows[step, :, r + 1:].any()
            assert (rows[step, :, lo:r + 1] > 0).all()
        assert np.allclose(mean, rows.mean(1), atol=1e-7)


def test_d2o_find_nearest_reference_case():
    """find_nearest_picks_most_similar_retained (crates/techniques/d2o/src/lib.rs:888-910) in spirit: with one head of
    dimension 2 the evicted row (1, 0) is nearest to the retained row pointing the same way; orthogonal and opposite rows
    lose; similarity of parallel rows is exactly 1."""
    k = np.zeros((1, 4, 2), dtype=np.float32)
    k[0, 0] = [1.0, 0.0]      # evicted
    k[0, 1] = [0.0, 1.0]      # orthogonal
    k[0, 2] = [2.0, 0.0]      # parallel
    k[0, 3] = [-1.0, 0.0]     # opposite
    pos, sim = orc.d2o_find_nearest(k, [0], [1, 2, 3])
    assert pos.tolist() == [2] and sim.tolist() == [1.0]
    pos, sim = orc.d2o_find_nearest(k, [0], [0])          # only itself: first of the list, similarity 0
    assert pos.tolist() == [0] and sim.tolist() == [0.0]
    pos, sim = orc.d2o_find_nearest(k, [0], [])
    assert pos.tolist() == [0] and sim.tolist() == [0.0]


def test_prefix_cache_file_layout_pins():
    """The byte layout stated in engine/src/session/prefix_cache.rs:1-30 and its FIXED_HEADER_BYTES = 100: the fixed
    header is 100 bytes, header_len counts everything after the header_len field up to the end of the token ids, the
    logits section sits between the token ids and the payload, and the payload is layer-major K then V."""
    k0 = np.arange(2 * 5 * 4, dtype=np.float16).reshape(2, 5, 4)
    v0 = -k0
    pay = orc.extract_packed_bytes(k0, 3) + orc.extract_packed_bytes(v0, 3)
    assert len(pay) == 2 * 2 * 3 * 4 * 2
    assert np.array_equal(np.frombuffer(pay[:48], dtype=np.float16), np.concatenate([k0[0, :3].ravel(), k0[1, :3].ravel()]))
    raw = orc.prefix_cache_encode(bytes(range(32)), bytes(range(32, 64)), [7, 8, 9], [0.5, -1.0], 3, 2, 4, [pay, pay])
    assert raw[:8] == b"ARGUSKV1" and int.from_bytes(raw[8:12], "little") == 2
    assert int.from_bytes(raw[12:16], "little") == 84 + 3 * 4                      # header_len
    assert raw[16:48] == bytes(range(32)) and int.from_bytes(raw[48:52], "little") == 3
    assert [int.from_bytes(raw[84 + 4 * i:88 + 4 * i], "little") for i in range(4)] == [2, 4, 2, 3]   # geometry, token_count
    assert len(raw) == 100 + 12 + 4 + 8 + 2 * len(pay)
    got = orc.prefix_cache_decode(raw, 2)
    assert got["token_ids"] == [7, 8, 9] and got["layers"] == [pay, pay] and got["last_logits"].tolist() == [0.5, -1.0]
    assert orc.prefix_cache_decode(b"ARGUSKV0" + raw[8:], 2) is None               # magic
    assert orc.prefix_cache_decode(raw[:8] + (1).to_bytes(4, "little") + raw[12:], 2) is None   # version 1 files are invalid
    assert orc.prefix_cache_decode(raw, 3) is None                                 # geometry mismatch
