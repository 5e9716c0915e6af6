"""KV write and eviction executors on the device against the numpy restatements of the reference's CPU code
(oracle.kv_scatter / compact_keep_positions / apply_weighted_merges): bit-exact, through the C ABI."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def be():
    from argus_engine_b200 import B200Backend

    return B200Backend(0)


def _cache(rng, hkv, cap, d, dtype):
    k = rng.standard_normal((hkv, cap, d)).astype(dtype)
    v = rng.standard_normal((hkv, cap, d)).astype(dtype)
    return k, v


@pytest.mark.parametrize("dtype", [np.float16, np.float32])
@pytest.mark.parametrize("S,write_pos", [(1, 0), (1, 77), (33, 5), (128, 384)])
def test_kv_scatter_bit_exact(be, dtype, S, write_pos):
    rng = np.random.default_rng(S + write_pos)
    hkv, cap, d = 8, 512, 128
    k, v = _cache(rng, hkv, cap, d, dtype)
    ks = (rng.standard_normal((S, hkv, d)) * 3).astype(np.float32)
    vs = (rng.standard_normal((S, hkv, d)) * 3).astype(np.float32)
    ks[0, 0, :4] = [65504.0, 65520.0, 1e-8, -0.0]   # F16 max, overflow to inf, underflow to zero, signed zero
    kd, vd = torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda()
    be.kv_scatter(torch.from_numpy(ks).cuda(), torch.from_numpy(vs).cuda(), kd, vd, write_pos)
    orc.kv_scatter(ks, vs, k, v, write_pos)
    assert np.array_equal(kd.cpu().numpy().view(np.uint8), k.view(np.uint8))
    assert np.array_equal(vd.cpu().numpy().view(np.uint8), v.view(np.uint8))


def test_kv_scatter_batched_one_row_per_sequence(be):
    """The decode-step form: one launch writes each sequence's new row at that sequence's own length."""
    rng = np.random.default_rng(21)
    hkv, d, lens, caps = 8, 128, [5, 1000, 77, 4095], [16, 1024, 128, 4096]
    ks = (rng.standard_normal((len(lens), hkv, d)) * 2).astype(np.float32)
    vs = (rng.standard_normal((len(lens), hkv, d)) * 2).astype(np.float32)
    caches = [_cache(rng, hkv, cap, d, np.float16) for cap in caps]
    kd = [torch.from_numpy(k).cuda() for k, _ in caches]
    vd = [torch.from_numpy(v).cuda() for _, v in caches]
    be.kv_scatter_batched(torch.from_numpy(ks).cuda(), torch.from_numpy(vs).cuda(), kd, vd, lens)
    for i, (k, v) in enumerate(caches):
        orc.kv_scatter(ks[i:i + 1], vs[i:i + 1], k, v, lens[i])
        assert np.array_equal(kd[i].cpu().numpy().view(np.uint8), k.view(np.uint8))
        assert np.array_equal(vd[i].cpu().numpy().view(np.uint8), v.view(np.uint8))
    with pytest.raises(RuntimeError):   # a full cache has no room for the row
        be.kv_scatter_batched(torch.from_numpy(ks).cuda(), torch.from_numpy(vs).cuda(), kd, vd, [5, 1000, 128, 10])


def test_kv_scatter_rejects_rows_outside_capacity(be):
    kd = torch.zeros(2, 16, 64, device="cuda", dtype=torch.float16)
    src = torch.zeros(4, 2, 64, device="cuda")
    with pytest.raises(RuntimeError):
        be.kv_scatter(src, src, kd, kd.clone(), 14)


def _h2o_like_keep(rng, cur, prefix, heavy, recent):
    cand = np.arange(prefix, cur - recent)
    hh = np.sort(rng.choice(cand, size=heavy, replace=False))
    return np.concatenate([np.arange(prefix), hh, np.arange(cur - recent, cur)]).astype(np.int32)


@pytest.mark.parametrize("dtype", [np.float16, np.float32])
@pytest.mark.parametrize("head", [-1, 3])
@pytest.mark.parametrize("cur,prefix,heavy,recent,write_start", [(1000, 4, 200, 64, 0), (4096, 0, 1500, 128, 0),
                                                                  (300, 10, 1, 5, 0), (2000, 0, 700, 100, 0)])
def test_kv_compact_matches_reference_shifts(be, dtype, head, cur, prefix, heavy, recent, write_start):
    rng = np.random.default_rng(cur + heavy)
    hkv, cap, d = 8, cur + 32, 128
    k, v = _cache(rng, hkv, cap, d, dtype)
    keep = _h2o_like_keep(rng, cur, prefix, heavy, recent)
    kd, vd = torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda()
    be.kv_compact(kd, vd, torch.from_numpy(keep).cuda(), write_start, head)
    h = None if head < 0 else head
    orc.compact_keep_positions(k, keep.tolist(), write_start, h)
    orc.compact_keep_positions(v, keep.tolist(), write_start, h)
    assert be.check_status() == 0
    assert np.array_equal(kd.cpu().numpy().view(np.uint8), k.view(np.uint8))
    assert np.array_equal(vd.cpu().numpy().view(np.uint8), v.view(np.uint8))


def test_kv_compact_in_chunks_and_edge_lists(be):
    """A scratch of 64 KB forces many passes (the order of the passes is what makes the in-place move safe); an empty
    list and an identity list move nothing; a list that would move a row to the right is refused through the status word."""
    from argus_engine_b200 import B200Backend

    small = B200Backend(0, workspace_bytes=64 << 10)
    rng = np.random.default_rng(9)
    hkv, cap, d = 4, 3000, 128
    k, v = _cache(rng, hkv, cap, d, np.float16)
    keep = _h2o_like_keep(rng, 2900, 8, 1200, 256)
    kd, vd = torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda()
    small.kv_compact(kd, vd, torch.from_numpy(keep).cuda(), 0)
    orc.compact_keep_positions(k, keep.tolist(), 0)
    orc.compact_keep_positions(v, keep.tolist(), 0)
    assert small.check_status() == 0
    assert np.array_equal(kd.cpu().numpy(), k) and np.array_equal(vd.cpu().numpy(), v)
    before = kd.clone()
    small.kv_compact(kd, vd, torch.zeros(0, dtype=torch.int32, device="cuda"), 0)
    small.kv_compact(kd, vd, torch.arange(100, dtype=torch.int32, device="cuda"), 0)
    assert small.check_status() == 0 and torch.equal(kd, before)
    small.kv_compact(kd, vd, torch.tensor([0, 1, 2], dtype=torch.int32, device="cuda"), 5)   # would move right
    assert small.check_status() == 2 and torch.equal(kd, before)
    # a source position at or beyond the cache's row count: the reference's slice index would panic; here the entry is
    # skipped (nothing is read out of bounds), the status word says so, and the other entries of the list still move
    small.kv_compact(kd, vd, torch.tensor([10, 20, cap, cap + 7], dtype=torch.int32, device="cuda"), 0)
    assert small.check_status() == 2
    assert torch.equal(kd[:, 0], before[:, 10]) and torch.equal(kd[:, 1], before[:, 20]) and torch.equal(kd[:, 2:], before[:, 2:])


@pytest.mark.parametrize("dtype", [np.float16, np.float32])
@pytest.mark.parametrize("axis", [0, 1, 2])
@pytest.mark.parametrize("d", [128, 66])   # 66: not a multiple of 4 channels, the one-channel-per-thread kernel
def test_kv_weighted_merge_bit_exact(be, dtype, axis, d):
    rng = np.random.default_rng(axis + 40)
    hkv, cap = 8, 700
    k, v = _cache(rng, hkv, cap, d, dtype)
    pos = rng.permutation(cap)
    merges, used = [], 0
    for m in range(60):
        n_from = int(rng.integers(0, 5))   # some merges have an empty list and leave their row alone
        into = int(pos[used])
        frm = [(int(pos[used + 1 + j]), float(rng.random() * 0.5)) for j in range(n_from)]
        used += 1 + n_from
        merges.append((into, float(0.5 + rng.random() * 0.5), frm))
    into_pos = np.array([m[0] for m in merges], dtype=np.int32)
    into_w = np.array([m[1] for m in merges], dtype=np.float32)
    from_start = np.cumsum([0] + [len(m[2]) for m in merges]).astype(np.int32)
    from_pos = np.array([p for m in merges for p, _ in m[2]], dtype=np.int32)
    from_w = np.array([w for m in merges for _, w in m[2]], dtype=np.float32)
    kd, vd = torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda()
    dev = lambda a: torch.from_numpy(a).cuda()
    be.kv_weighted_merge(kd, vd, dev(into_pos), dev(into_w), dev(from_start), dev(from_pos), dev(from_w), axis)
    orc.apply_weighted_merges(k, v, [(m[0], np.float32(m[1]), [(p, np.float32(w)) for p, w in m[2]]) for m in merges], axis)
    assert np.array_equal(kd.cpu().numpy().view(np.uint8), k.view(np.uint8))
    assert np.array_equal(vd.cpu().numpy().view(np.uint8), v.view(np.uint8))


@pytest.mark.parametrize("hq,hkv,d", [(8, 2, 128), (4, 4, 64), (32, 8, 128)])
@pytest.mark.parametrize("S,q_start,q_window", [(40, 0, 32), (6, 0, 3), (17, 300, 8), (5, 0, 9)])
def test_prefill_attention_scores_vs_reference_restatement(be, hq, hkv, d, S, q_start, q_window):
    """The H2O prefill seed (engine/src/kv/standard_format.rs:1400-1510): summed, per-row and head-mean outputs of the
    trailing query window against the step-by-step restatement, at the score tolerance of the decode tests; the summed
    output is bit-identical to the sum of the per-row output in row order (the reference's cross-check, section 3b)."""
    rng = np.random.default_rng(hq * 1000 + S + q_start)
    T = q_start + S
    cap = T + 11
    q = (rng.standard_normal((S, hq, d)) * 0.8).astype(np.float32)
    k = rng.standard_normal((hkv, cap, d)).astype(np.float16)
    v = rng.standard_normal((hkv, cap, d)).astype(np.float16)
    want_sum, want_rows, want_mean = orc.prefill_attention_scores(q, k, hkv, q_start, q_window, T)
    qwin = min(q_window, S)
    dev = lambda a: torch.from_numpy(a).cuda()
    qd, kd, vd = dev(q), dev(k), dev(v)
    sum_out = torch.zeros(hq, T, device="cuda")
    rows = torch.zeros(qwin, hq, T, device="cuda")
    be.prefill_attention_scores(qd, kd, vd, T, q_start, q_window, sum_out=sum_out, per_row=rows, per_row_per_head=True)
    mean = torch.zeros(qwin, T, device="cuda")
    sum2 = torch.zeros(hq, T, device="cuda")
    be.prefill_attention_scores(qd, kd, vd, T, q_start, q_window, sum_out=sum2, per_row=mean, per_row_per_head=False)
    assert be.check_status() == 0
    tol = dict(atol=1e-7, rtol=1e-2)
    np.testing.assert_allclose(rows.cpu().numpy(), want_rows, **tol)
    np.testing.assert_allclose(sum_out.cpu().numpy(), want_sum, atol=1e-6, rtol=1e-2)
    np.testing.assert_allclose(mean.cpu().numpy(), want_mean, atol=1e-7, rtol=1e-2)
    assert torch.equal(sum_out, sum2)                      # the staged route gives the same bits as the direct one
    acc = torch.zeros(hq, T, device="cuda")
    for r in range(qwin):
        acc = acc + rows[r]
    assert torch.equal(acc, sum_out)
    assert np.allclose(rows.cpu().numpy().sum(-1), 1.0, atol=1e-5)   # each row is a distribution over keys 0..=p
    # the keep list an eviction would compute from the seed is the one the reference's scores give
    flat = sum_out.sum(0).cpu().numpy()
    heavy = max(1, T // 8)
    assert orc.keep_top_k(T, 2, 4, heavy, flat) == orc.keep_top_k(T, 2, 4, heavy, want_sum.sum(0)) or T < 16


@pytest.mark.parametrize("window", [0, 16])
def test_prefill_attention_scores_ignores_stale_per_row_contents(be, window):
    """The per-row buffer arrives full of NaN (a reused or uninitialised buffer). The reference assigns keys lo..=p of
    each row and adds only those into the sums, so entries outside a row's range must never reach sum_out."""
    rng = np.random.default_rng(3 + window)
    hq, hkv, d, S, q_start, qw = 8, 2, 128, 40, 60, 12
    T = q_start + S
    q = (rng.standard_normal((S, hq, d)) * 0.8).astype(np.float32)
    k = rng.standard_normal((hkv, T, d)).astype(np.float16)
    v = rng.standard_normal((hkv, T, d)).astype(np.float16)
    want_sum, want_rows, _ = orc.prefill_attention_scores(q, k, hkv, q_start, qw, T, window or None)
    dev = lambda a: torch.from_numpy(a).cuda()
    sum_out = torch.zeros(hq, T, device="cuda")
    rows = torch.full((qw, hq, T), float("nan"), device="cuda")
    be.prefill_attention_scores(dev(q), dev(k), dev(v), T, q_start, qw, sum_out=sum_out, per_row=rows, window=window)
    assert be.check_status() == 0
    np.testing.assert_allclose(sum_out.cpu().numpy(), want_sum, atol=1e-6, rtol=1e-2)
    got = rows.cpu().numpy()
    for r in range(qw):
        p = q_start + S - qw + r
        lo = max(0, p - (window - 1)) if window else 0
        np.testing.assert_allclose(got[r, :, lo:p + 1], want_rows[r, :, lo:p + 1], atol=1e-7, rtol=1e-2)
        assert np.isnan(got[r, :, p + 1:]).all() and np.isnan(got[r, :, :lo]).all()   # left as found


@pytest.mark.parametrize("window", [4, 64, 1000])
def test_prefill_attention_scores_sliding_window(be, window):
    """Sliding-window band (engine/src/kv/standard_format.rs:1455-1461): row at position p sees keys
    max(0, p - (w-1))..=p; keys outside a row's band stay zero."""
    rng = np.random.default_rng(window)
    hq, hkv, d, S, q_start, qw = 8, 2, 128, 70, 130, 16
    T = q_start + S
    q = (rng.standard_normal((S, hq, d)) * 0.8).astype(np.float32)
    k = rng.standard_normal((hkv, T + 8, d)).astype(np.float16)
    v = rng.standard_normal((hkv, T + 8, d)).astype(np.float16)
    want_sum, want_rows, want_mean = orc.prefill_attention_scores(q, k, hkv, q_start, qw, T, window)
    dev = lambda a: torch.from_numpy(a).cuda()
    sum_out = torch.zeros(hq, T, device="cuda")
    rows = torch.zeros(qw, hq, T, device="cuda")
    be.prefill_attention_scores(dev(q), dev(k), dev(v), T, q_start, qw, sum_out=sum_out, per_row=rows, window=window)
    mean = torch.zeros(qw, T, device="cuda")
    be.prefill_attention_scores(dev(q), dev(k), dev(v), T, q_start, qw, per_row=mean, per_row_per_head=False, window=window)
    assert be.check_status() == 0
    np.testing.assert_allclose(rows.cpu().numpy(), want_rows, atol=1e-7, rtol=1e-2)
    np.testing.assert_allclose(sum_out.cpu().numpy(), want_sum, atol=1e-6, rtol=1e-2)
    np.testing.assert_allclose(mean.cpu().numpy(), want_mean, atol=1e-7, rtol=1e-2)
    assert (rows.cpu().numpy() != 0).sum() == (want_rows != 0).sum()   # nothing written outside the bands


@pytest.mark.parametrize("dtype", [np.float16, np.float32])
@pytest.mark.parametrize("hkv,d,n_e,n_r", [(8, 128, 70, 333), (2, 64, 5, 40), (4, 128, 33, 1)])
def test_d2o_nearest_bit_exact(be, dtype, hkv, d, n_e, n_r):
    """D2O Eq. 8 (crates/techniques/d2o/src/lib.rs:187-255): the selected retained position and the similarity of every
    evicted position equal the step-by-step restatement bit for bit - including exact ties (duplicated rows: the first
    in list order wins), an evicted position that also sits in the retained list (skipped) and an all-zero row."""
    rng = np.random.default_rng(n_e * 7 + n_r)
    cap = 1024
    k = rng.standard_normal((hkv, cap, d)).astype(dtype)
    pos = rng.permutation(cap)
    evict = pos[:n_e].astype(np.int32)
    retain = np.sort(pos[n_e:n_e + n_r]).astype(np.int32)
    if n_r >= 40:
        k[:, retain[7]] = k[:, retain[3]]          # an exact tie between two retained rows
        k[:, evict[0]] = k[:, retain[3]] * dtype(0.5)   # ... which the first evicted row points at
        k[:, retain[11]] = 0                       # zero norm: similarity 0 by the denominator guard
        retain[20] = evict[1]                      # an evicted position inside the retained list is skipped
    want_pos, want_sim = orc.d2o_find_nearest(k, evict, retain)
    dev = lambda a: torch.from_numpy(a).cuda()
    got_pos, got_sim = be.d2o_nearest(dev(k), dev(evict), dev(retain))
    assert np.array_equal(got_pos.cpu().numpy(), want_pos)
    assert np.array_equal(got_sim.cpu().numpy().view(np.uint32), want_sim.view(np.uint32))
    if n_r >= 40:
        assert want_pos[0] == retain[3] and want_pos[1] != evict[1]


def test_d2o_nearest_empty_lists(be):
    k = torch.randn(2, 64, 64, device="cuda").half()
    ev = torch.tensor([5, 9], dtype=torch.int32, device="cuda")
    none = torch.zeros(0, dtype=torch.int32, device="cuda")
    pos, sim = be.d2o_nearest(k, ev, none)
    assert pos.tolist() == [5, 9] and sim.tolist() == [0.0, 0.0]          # empty retained list: itself, similarity 0
    pos, sim = be.d2o_nearest(k, ev, torch.tensor([5], dtype=torch.int32, device="cuda"))
    assert pos.tolist()[0] == 5 and sim.tolist()[0] == 0.0                 # only itself to choose from
    pos, sim = be.d2o_nearest(k, none, ev)
    assert pos.numel() == 0


@pytest.mark.parametrize("dtype", [np.float16, np.float32])
@pytest.mark.parametrize("seq_major", [False, True])
@pytest.mark.parametrize("host_side", ["device", "pinned"])
def test_prefix_cache_payload_round_trip(be, dtype, seq_major, host_side):
    """Session prefix cache (engine/src/session/prefix_cache.rs): the per-layer payload written from a device-resident
    cache is byte-identical to what the reference's snapshot_prefix packs on the host; a two-layer ARGUSKV1 v2 file built
    around it parses back; restoring the payload into a cache of another capacity reproduces the prefix rows bit for bit
    and leaves the rows behind them alone."""
    rng = np.random.default_rng(12)
    hkv, cap, d, tc = 4, 300, 128, 173
    layers = []
    for layer in range(2):
        k, v = _cache(rng, hkv, cap, d, dtype)
        kd, vd = torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda()
        if seq_major:   # the same values laid out [cap, Hkv, D]
            kd, vd = kd.transpose(0, 1).contiguous(), vd.transpose(0, 1).contiguous()
        nbytes = 2 * hkv * tc * d * k.itemsize
        dst = torch.zeros(nbytes, dtype=torch.uint8, device="cuda") if host_side == "device" else torch.zeros(nbytes, dtype=torch.uint8).pin_memory()
        be.kv_snapshot_prefix(kd, vd, hkv, tc, dst)
        torch.cuda.synchronize()
        want = orc.extract_packed_bytes(k, tc) + orc.extract_packed_bytes(v, tc)
        assert bytes(dst.cpu().numpy()) == want
        layers.append((k, v, want))
    raw = orc.prefix_cache_encode(b"m" * 32, b"t" * 32, range(tc), [1.0, 2.0], 0, hkv, d, [p for _, _, p in layers])
    parsed = orc.prefix_cache_decode(raw, 2)
    assert parsed is not None and parsed["layers"] == [p for _, _, p in layers]
    for (k, v, _), payload in zip(layers, parsed["layers"]):
        cap2 = 256
        filler = 3.0
        k2 = torch.full((hkv, cap2, d), filler, dtype=torch.from_numpy(k).dtype, device="cuda")
        v2 = torch.full_like(k2, filler)
        if seq_major:
            k2, v2 = k2.transpose(0, 1).contiguous(), v2.transpose(0, 1).contiguous()
        src = torch.frombuffer(bytearray(payload), dtype=torch.uint8)
        src = src.cuda() if host_side == "device" else src.pin_memory()
        be.kv_restore_prefix(k2, v2, hkv, tc, src)
        torch.cuda.synchronize()
        k2h, v2h = (t.transpose(0, 1) if seq_major else t for t in (k2, v2))
        assert np.array_equal(k2h[:, :tc].cpu().numpy().view(np.uint8), np.ascontiguousarray(k[:, :tc]).view(np.uint8))
        assert np.array_equal(v2h[:, :tc].cpu().numpy().view(np.uint8), np.ascontiguousarray(v[:, :tc]).view(np.uint8))
        assert (k2h[:, tc:] == filler).all() and (v2h[:, tc:] == filler).all()
    assert be.check_status() == 0


def test_managed_kv_buffers_are_made_resident_and_decoded(be):
    """KV residency: the engine's CUDA backend allocates KV as managed memory (engine/src/backend/cuda_pc/memory.rs:36-44).
    A managed buffer filled from the host, advised and prefetched once (argus_b200_kv_make_resident), decodes to the same
    result as device memory; a device pointer is accepted as is, a host pointer is declined."""
    import ctypes as C

    from argus_engine_b200 import ArgusB200Error, workloads as wl

    hq, hkv, d, T = 32, 8, 128, 6000
    case = wl.decode_case(31, [T], hq, hkv, d)
    nbytes = case.k[0].nbytes
    ptrs = [be.kv_alloc(nbytes, managed=True) for _ in range(2)]
    for ptr, arr in zip(ptrs, (case.k[0], case.v[0])):   # the host writes the pages, as a CPU-side cache fill would
        C.memmove(ptr, arr.ctypes.data, nbytes)
        be.kv_make_resident(ptr, nbytes)
    q = torch.from_numpy(case.q[0]).cuda()
    out = torch.zeros(hq, d, device="cuda")
    rc = be._lib.argus_b200_attention_gen(be._h, be._stream(), q.data_ptr(), C.c_void_p(ptrs[0]), C.c_void_p(ptrs[1]), out.data_ptr(),
                                          hq, hkv, d, T, 1, T * d, d, None)
    assert rc == 0
    torch.cuda.synchronize()
    want, _ = orc.attention_gen(case.q[0], case.k[0].view(np.uint16), case.v[0].view(np.uint16), hq, hkv, d, T)
    np.testing.assert_allclose(out.cpu().numpy(), want, atol=2e-3, rtol=1e-2)
    be.kv_make_resident(q.data_ptr(), q.numel() * 4)          # device memory: nothing to do
    host = torch.zeros(16)
    with pytest.raises(ArgusB200Error):
        be.kv_make_resident(host.data_ptr(), 64)
    for ptr in ptrs:
        be.kv_free(ptr)
