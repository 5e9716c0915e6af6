"""The benchmarked workloads at their FULL sizes through the C ABI (batched F16 decode B=16, one-million-token decode,
KIVI Q4 decode B=8 x 32768 with the H2O vector, BF16 causal prefill B=4 x 4096): against the CPU oracle where it
finishes in seconds, and through size-independent properties of the domain (a split/sharded result equals the unsplit
one, probabilities sum to one, a merge of partials equals the whole, an attention output lies in the convex hull of
the visible V rows)."""
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

    b = B200Backend(0, workspace_bytes=256 << 20)
    yield b
    b.close()


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_batched_decode_full_batch_vs_oracle(be):
    """The batched decode as benchmarked (B=16, Hq=32, Hkv=8, D=128, lengths U[1024,8192], seed 1): 16 sequences in ONE
    launch, every sequence against the oracle."""
    case = wl.config2()
    B = len(case.lens)
    out = torch.full((B, 32, 128), float("nan"), device="cuda")
    be.attention_gen_batched(_dev(case.q), [_dev(k) for k in case.k], [_dev(v) for v in case.v], case.lens, out, 32, 8, 128)
    got = out.cpu().numpy()
    for i in range(B):
        want, _ = orc.attention_gen(case.q[i], case.k[i].view(np.uint16), case.v[i].view(np.uint16), 32, 8, 128,
                                    case.lens[i], avx2=True)
        np.testing.assert_allclose(got[i], want, atol=OUT_ATOL, rtol=OUT_RTOL)
    assert be.check_status() == 0


def test_one_million_token_decode(be):
    """The long-context decode shape: Hq=64, Hkv=8, D=128, T=2^20 on one GPU (4.3 GB of K/V). (1) the 8 query heads of one KV head against
    the oracle run on that head's 1M rows; (2) the result equals the (o, lse) merge of 8 sequence shards, each decoded
    on its own - the algebra the multi-GPU path relies on; (3) the lse equals the oracle's log-sum-exp."""
    from argus_engine_b200 import DecodeExtras

    T, hq, hkv, d = 1 << 20, 64, 8, 128
    gen = torch.Generator(device="cuda").manual_seed(11)
    k = torch.randn(hkv, T, d, device="cuda", generator=gen).to(torch.float16)
    v = torch.randn(hkv, T, d, device="cuda", generator=gen).to(torch.float16)
    q = torch.randn(hq, d, device="cuda", generator=gen)
    out = torch.zeros(hq, d, device="cuda")
    ex = DecodeExtras(lse=torch.zeros(hq, device="cuda"))
    be.attention_gen(q, k, v, out, hq, hkv, d, T, extras=ex)
    torch.cuda.synchronize()
    assert be.check_status() == 0
    # (1) oracle on KV head 3 (query heads 24..31)
    kvh, g = 3, hq // hkv
    kh = k[kvh:kvh + 1].cpu().numpy().view(np.uint16)
    vh = v[kvh:kvh + 1].cpu().numpy().view(np.uint16)
    qh = q[kvh * g:(kvh + 1) * g].cpu().numpy()
    want, want_p = orc.attention_gen(qh, kh, vh, g, 1, d, T, want_scores=True)
    np.testing.assert_allclose(out[kvh * g:(kvh + 1) * g].cpu().numpy(), want, atol=OUT_ATOL, rtol=OUT_RTOL)
    # (3) lse = ln sum exp(s): from the oracle's probabilities of the maximal logit, p_max = exp(s_max - lse)
    s_max = (kh.view(np.float16).astype(np.float32)[0] @ qh.T / np.sqrt(d)).max(0)
    np.testing.assert_allclose(ex.lse[kvh * g:(kvh + 1) * g].cpu().numpy(), s_max - np.log(want_p.max(1)), atol=2e-3)
    # (2) eight shards, merged
    N = 8
    parts = torch.zeros(N, hq * d + hq, device="cuda")
    for r in range(N):
        lo, hi = r * (T // N), (r + 1) * (T // N)
        po = parts[r, :hq * d].view(hq, d)
        pex = DecodeExtras(lse=parts[r, hq * d:])
        be.attention_gen(q, k[:, lo:hi], v[:, lo:hi], po, hq, hkv, d, hi - lo, extras=pex)
    merged = torch.zeros(hq, d, device="cuda")
    mlse = torch.zeros(hq, device="cuda")
    be.lse_merge(parts, hq, d, merged, mlse)
    torch.cuda.synchronize()
    np.testing.assert_allclose(merged.cpu().numpy(), out.cpu().numpy(), atol=2e-5, rtol=1e-4)
    np.testing.assert_allclose(mlse.cpu().numpy(), ex.lse.cpu().numpy(), atol=1e-4)


def test_kivi_full_length_sequence(be):
    """The KIVI Q4 workload, one of its eight sequences at full length (T=32768: 255 flushes + 128 residual tokens) packed by
    the device container: the decode output and the fused H2O group-mean vector against the oracle on the same bytes;
    the vector sums to one per KV head (each of its g rows is a distribution)."""
    from argus_engine_b200 import DecodeExtras
    from argus_engine_b200.kivi_cache import KiviDeviceCache

    T, hq, hkv, d = 32768, 32, 8, 128
    src = wl.kivi_source(2, [T], hq, hkv, d, 128, 4)
    cache = KiviDeviceCache(be, hkv, d, T, 128, 4)
    cache.update(_dev(src.k[0]), _dev(src.v[0]))
    qk, qv, rk, rv, qt, rt = cache.seq(res_f16=False)
    out = torch.zeros(1, hq, d, device="cuda")
    ex = DecodeExtras(head_scores=torch.zeros(1, hkv, T, device="cuda"), score_stride=T)
    be.kivi_attention_batched(_dev(src.q), [(qk, qv, rk, rv, qt, rt)], out, hq, hkv, d, 128, 4, 1 / np.sqrt(d), extras=ex)
    torch.cuda.synchronize()
    assert be.check_status() == 0
    vk, vv = orc.kivi_assemble_view(qk.cpu().numpy(), qv.cpu().numpy(), rk.cpu().numpy(), rv.cpu().numpy(), hkv, d, 128, 4,
                                    qt, rt)
    want, want_p = orc.attention_gen(src.q[0], vk, vv, hq, hkv, d, T, head_major=False, want_scores=True)
    np.testing.assert_allclose(out[0].cpu().numpy(), want, atol=OUT_ATOL, rtol=OUT_RTOL)
    sh = np.zeros(hkv * T, dtype=np.float32)
    orc.score_accumulate_layer(want_p, T, hq, hkv, T, np.zeros(T, dtype=np.float32), sh)
    got = ex.head_scores[0].cpu().numpy()
    np.testing.assert_allclose(got, sh.reshape(hkv, T), atol=P_ATOL, rtol=P_RTOL)
    np.testing.assert_allclose(got.sum(1), 1.0, atol=1e-4)


def test_kivi_full_batch_as_benchmarked(be):
    """The KIVI Q4 decode exactly as the benchmark launches it: B=8 sequences of 32768 tokens (seed 2, 1 % of the K
    channels scaled by 8), F16 residual window, ONE launch with the fused [8, 8, 32768] group-mean vector. Two of the
    eight sequences against the oracle on the same packed bytes (output and vector); for all eight every KV head's
    vector sums to one and every output row lies inside the range of the dequantised V values."""
    from argus_engine_b200 import DecodeExtras
    from argus_engine_b200.kivi_cache import KiviDeviceCache

    src = wl.config3_source()
    B, T, hq, hkv, d = len(src.k), src.k[0].shape[0], 32, 8, 128
    seqs = []
    for i in range(B):
        cache = KiviDeviceCache(be, hkv, d, T, 128, 4)
        cache.update(_dev(src.k[i]), _dev(src.v[i]))
        seqs.append(cache.seq(res_f16=True))
    out = torch.full((B, hq, d), float("nan"), device="cuda")
    ex = DecodeExtras(head_scores=torch.zeros(B, hkv, T, device="cuda"), score_stride=T)
    be.kivi_attention_batched(_dev(src.q), seqs, out, hq, hkv, d, 128, 4, 1 / np.sqrt(d), res_f16=True, extras=ex)
    torch.cuda.synchronize()
    assert be.check_status() == 0
    got, got_s = out.cpu().numpy(), ex.head_scores.cpu().numpy()
    np.testing.assert_allclose(got_s.sum(-1), 1.0, atol=1e-4)
    vmax = max(float(np.abs(v).max()) for v in src.v)
    assert np.isfinite(got).all() and np.abs(got).max() <= vmax * 1.07 + 1e-3   # Q4 blocks stay within their group's range
    for i in (0, B - 1):
        qk, qv, rk, rv, qt, rt = seqs[i]
        vk, vv = orc.kivi_assemble_view(qk.cpu().numpy(), qv.cpu().numpy(), rk.float().cpu().numpy(), rv.float().cpu().numpy(),
                                        hkv, d, 128, 4, qt, rt)
        want, want_p = orc.attention_gen(src.q[i], vk, vv, hq, hkv, d, T, head_major=False, want_scores=True, avx2=True)
        np.testing.assert_allclose(got[i], want, atol=OUT_ATOL, rtol=OUT_RTOL)
        sh = np.zeros(hkv * T, dtype=np.float32)
        orc.score_accumulate_layer(want_p, T, hq, hkv, T, np.zeros(T, dtype=np.float32), sh)
        np.testing.assert_allclose(got_s[i], sh.reshape(hkv, T), atol=P_ATOL, rtol=P_RTOL)


def test_prefill_full_size_bf16(be):
    """The causal prefill at its benchmarked size: B=4, S=4096, Hq=32, Hkv=8, D=128, BF16 in and out, seed 3, drawn by the
    seeded host generator. Four (batch, head) pairs - first and last batch, first and last head group - against the
    oracle's tiled F32 prefill on the BF16-rounded inputs (all 4096 rows each), compared after rounding the oracle to
    BF16; every output row of every pair lies in the convex hull of its visible V rows (|o| <= running max |v|), and row 0
    of every head equals V row 0 exactly."""
    B, S, hq, hkv, d = 4, 4096, 32, 8, 128
    case = wl.config4(B, S)
    q = _dev(case.q).to(torch.bfloat16)
    k = _dev(case.k).to(torch.bfloat16)
    v = _dev(case.v).to(torch.bfloat16)
    out = torch.full((B, S, hq, d), float("nan"), dtype=torch.bfloat16, device="cuda")
    assert be.flash_attention_prefill(q, k, v, out, hq, hkv, S, S, d, S, B, True)
    torch.cuda.synchronize()
    assert be.check_status() == 0
    got = out.float().cpu().numpy()
    assert np.isfinite(got).all()
    g = hq // hkv
    hull = np.maximum.accumulate(np.abs(case.v), axis=2)           # [B, Hkv, S, D]: running max |v| over visible keys
    bound = hull.transpose(0, 2, 1, 3).repeat(g, axis=2)            # [B, S, Hq, D]
    assert (np.abs(got) <= bound * (1 + 2.0 ** -7) + 1e-6).all()
    np.testing.assert_array_equal(got[:, 0], case.v[:, :, 0].repeat(g, axis=1))
    for bh in (0, hq - 1, 2 * hq + 13, (B - 1) * hq + hq - 1):
        want = orc.flash_prefill(case.q, case.k, case.v, hq, hkv, S, S, d, S, bh_range=(bh, bh + 1))
        b, h = divmod(bh, hq)
        np.testing.assert_allclose(got[b, :, h], wl._round_bf16(want[b, :, h]), atol=OUT_ATOL, rtol=OUT_RTOL + 2.0 ** -8)
