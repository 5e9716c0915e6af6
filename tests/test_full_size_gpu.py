"""The benchmark configurations at their FULL sizes (BASELINE configs[1], [2], [4]) through the C ABI: against the
CPU oracle where it finishes in seconds, and through size-independent properties of the domain (a split/sharded
result equals the unsplit one, probabilities sum to one, a merge of partials equals the whole)."""
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


def test_config2_full_batch_vs_oracle(be):
    """configs[1] as benchmarked: 16 sequences of 1024..8192 tokens in ONE launch, every sequence against the oracle."""
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


def test_config5_one_million_tokens(be):
    """configs[4]: Hq=64, Hkv=8, D=128, T=2^20 on one GPU (4.3 GB of K/V). (1) the 8 query heads of one KV head against
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


def test_config3_full_length_sequence(be):
    """configs[2], one of its eight sequences at full length (T=32768: 255 flushes + 128 residual tokens, Q4) packed by
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
