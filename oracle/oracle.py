"""ctypes front end of the CPU oracle (``oracle/argus_oracle.cpp``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by the benchmark's
CPU-baseline leg. The shipped package never imports it.

Each wrapper takes/returns numpy arrays; shapes and strides follow the reference's conventions
(K/V HeadMajor ``[Hkv, cap, D]`` or SeqMajor ``[T, Hkv, D]``; see the C++ file for the reference
lines each function restates).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libargus_oracle.so")


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside it (g++ only; a few seconds)."""
    src = os.path.join(_HERE, "argus_oracle.cpp")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "libargus_oracle.so"], stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_SO)
        _lib.orc_kivi_new.restype = C.c_void_p
        for n in ("orc_kivi_q_tokens", "orc_kivi_res_tokens", "orc_kivi_qk_bytes", "orc_kivi_qv_bytes",
                  "orc_keep_top_k", "orc_h2o_keep"):
            getattr(_lib, n).restype = C.c_long
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def num_threads() -> int:
    return int(lib().orc_num_threads())


def f32_to_f16_bits(x: np.ndarray) -> np.ndarray:
    x = _f32(x)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().orc_f32_to_f16(_p(x), _p(out), C.c_long(x.size))
    return out


def lcg(n: int, seed: int) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    lib().orc_lcg_gen(_p(out), C.c_long(n), C.c_uint32(seed))
    return out


def _kv_args(k: np.ndarray, head_major: bool, hkv: int, d: int):
    """Element strides (head_stride, pos_stride) for a contiguous K/V array."""
    if head_major:  # [Hkv, cap, D]
        cap = k.shape[-2]
        return cap * d, d
    return d, hkv * d  # [T, Hkv, D]


def attention_gen(q, k, v, hq, hkv, d, T, head_major=True, want_scores=False, score_stride=None,
                  guards=False, avx2=False, n_threads=0):
    """Single-query GQA decode. k/v: float32 or uint16 (F16 bits). Returns (out[hq,d], scores|None)."""
    q = _f32(q).reshape(hq, d)
    is_f16 = k.dtype == np.uint16 or k.dtype == np.float16
    k = np.ascontiguousarray(k)
    v = np.ascontiguousarray(v)
    hs, ps = _kv_args(k, head_major, hkv, d)
    out = np.zeros((hq, d), dtype=np.float32)
    scores = None
    stride = 0
    if want_scores:
        stride = int(score_stride or T)
        scores = np.zeros((hq, stride), dtype=np.float32)
    if avx2:
        rc = lib().orc_attention_gen_avx2(_p(q), _p(k), _p(v), int(is_f16), _p(out), hq, hkv, d, C.c_long(T),
                                          C.c_long(hs), C.c_long(ps), _p(scores), C.c_long(stride),
                                          int(n_threads))
    else:
        rc = lib().orc_attention_gen(_p(q), _p(k), _p(v), int(is_f16), _p(out), hq, hkv, d, C.c_long(T),
                                     C.c_long(hs), C.c_long(ps), _p(scores), C.c_long(stride), int(guards))
    if rc != 0:
        raise ValueError("oracle attention_gen rejected the arguments")
    return out, scores


def flash_prefill(q, k, v, hq, hkv, S, T, d, cap, head_major=True, br=32, bc=32, window=0,
                  bh_range=None, n_threads=0):
    """Causal GQA prefill. q: [B,S,Hq,D] f32; k/v f32 [B,Hkv,cap,D] (HeadMajor) or [B,cap,Hkv,D]."""
    q = _f32(q)
    k = _f32(k)
    v = _f32(v)
    B = q.shape[0]
    out = np.zeros_like(q)
    b0, b1 = bh_range if bh_range else (0, 0)
    rc = lib().orc_flash_prefill(_p(q), _p(k), _p(v), _p(out), B, hq, hkv, C.c_long(S), C.c_long(T), d,
                                 C.c_long(cap), int(head_major), br, bc, C.c_long(window), C.c_long(b0),
                                 C.c_long(b1), int(n_threads))
    if rc != 0:
        raise ValueError("oracle flash_prefill rejected the arguments")
    return out


def block_bytes(bits: int) -> int:
    return int(lib().orc_kv_block_bytes(bits))


def kv_quantize(x: np.ndarray, bits: int) -> np.ndarray:
    x = _f32(x).reshape(-1)
    assert x.size % 32 == 0
    nb = x.size // 32
    out = np.zeros(nb * block_bytes(bits), dtype=np.uint8)
    assert lib().orc_kv_quantize(_p(x), C.c_long(nb), bits, _p(out)) == 0
    return out


def kv_dequantize(blocks: np.ndarray, bits: int) -> np.ndarray:
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    nb = blocks.size // block_bytes(bits)
    out = np.zeros(nb * 32, dtype=np.float32)
    assert lib().orc_kv_dequantize(_p(blocks), C.c_long(nb), bits, _p(out)) == 0
    return out


class KiviCache:
    """Restated quantized recent-window container (ring + flush + view)."""

    def __init__(self, hkv: int, d: int, res_cap: int, bits: int):
        self.hkv, self.d, self.res_cap, self.bits = hkv, d, res_cap, bits
        self._h = C.c_void_p(lib().orc_kivi_new(hkv, d, res_cap, bits))
        if not self._h:
            raise ValueError("bad KIVI geometry")

    def __del__(self):
        if getattr(self, "_h", None):
            lib().orc_kivi_free(self._h)
            self._h = None

    def update(self, new_k: np.ndarray, new_v: np.ndarray) -> None:
        new_k = _f32(new_k).reshape(-1, self.hkv, self.d)
        new_v = _f32(new_v).reshape(-1, self.hkv, self.d)
        lib().orc_kivi_update(self._h, _p(new_k), _p(new_v), C.c_long(new_k.shape[0]))

    @property
    def q_tokens(self) -> int:
        return int(lib().orc_kivi_q_tokens(self._h))

    @property
    def res_tokens(self) -> int:
        return int(lib().orc_kivi_res_tokens(self._h))

    def export(self):
        """(qk bytes, qv bytes, res_k [Hkv,res_cap,D], res_v) as the device kernels index them."""
        qk = np.zeros(int(lib().orc_kivi_qk_bytes(self._h)), dtype=np.uint8)
        qv = np.zeros(int(lib().orc_kivi_qv_bytes(self._h)), dtype=np.uint8)
        rk = np.zeros((self.hkv, self.res_cap, self.d), dtype=np.float32)
        rv = np.zeros_like(rk)
        lib().orc_kivi_export(self._h, _p(qk), _p(qv), _p(rk), _p(rv))
        return qk, qv, rk, rv


def kivi_assemble_view(qk, qv, res_k, res_v, hkv, d, res_cap, bits, q_tokens, res_tokens):
    """F32 SeqMajor [T,Hkv,D] K and V views from raw container buffers."""
    T = q_tokens + res_tokens
    vk = np.zeros((T, hkv, d), dtype=np.float32)
    vv = np.zeros((T, hkv, d), dtype=np.float32)
    qk = np.ascontiguousarray(qk, dtype=np.uint8)
    qv = np.ascontiguousarray(qv, dtype=np.uint8)
    res_k = _f32(res_k)
    res_v = _f32(res_v)
    rc = lib().orc_kivi_assemble_view(_p(qk), _p(qv), _p(res_k), _p(res_v), hkv, d, res_cap, bits,
                                      C.c_long(q_tokens), C.c_long(res_tokens), _p(vk), _p(vv))
    assert rc == 0
    return vk, vv


def score_accumulate_layer(scores, T, hq, hkv, max_seq, step_flat, step_head, score_offset=0):
    scores = _f32(scores)
    stride = scores.shape[-1]
    lib().orc_score_accumulate_layer(_p(scores), C.c_long(stride), C.c_long(T), hq, hkv,
                                     C.c_long(score_offset), C.c_long(max_seq), _p(step_flat), _p(step_head))


def score_begin_step(importance, head_importance, step_flat, step_head, hkv, max_seq, decay):
    lib().orc_score_begin_step(_p(importance), _p(head_importance), _p(step_flat), _p(step_head), hkv,
                               C.c_long(max_seq), C.c_float(decay))


def score_end_step(importance, head_importance, step_flat, step_head, hkv, max_seq):
    lib().orc_score_end_step(_p(importance), _p(head_importance), _p(step_flat), _p(step_head), hkv,
                             C.c_long(max_seq))


def score_fused_reduce(scores, importance, head_importance, decay_factor, n_layers, hq, hkv, T,
                       score_stride, max_seq):
    scores = _f32(scores)
    lib().orc_score_fused_reduce(_p(scores), _p(importance), _p(head_importance), C.c_float(decay_factor),
                                 n_layers, hq, hkv, C.c_long(T), C.c_long(score_stride), C.c_long(max_seq))


def score_reduce_per_layer(scores, layer_flat, decay_factor, n_layers, hq, T, score_stride, max_seq):
    scores = _f32(scores)
    lib().orc_score_reduce_per_layer(_p(scores), _p(layer_flat), C.c_float(decay_factor), n_layers, hq,
                                     C.c_long(T), C.c_long(score_stride), C.c_long(max_seq))


def keep_top_k(current, prefix, recent, heavy, score=None):
    keep = np.zeros(max(current, 1), dtype=np.int64)
    s = None if score is None else _f32(score)
    n = lib().orc_keep_top_k(C.c_long(current), C.c_long(prefix), C.c_long(recent), C.c_long(heavy), _p(s),
                             C.c_long(0 if s is None else s.size), _p(keep))
    return keep[:n].tolist()


def h2o_keep(current, protected_prefix, hh_size, recent_size, score=None):
    keep = np.zeros(max(current, 1), dtype=np.int64)
    s = None if score is None else _f32(score)
    n = lib().orc_h2o_keep(C.c_long(current), C.c_long(protected_prefix), C.c_long(hh_size),
                           C.c_long(recent_size), _p(s), C.c_long(0 if s is None else s.size), _p(keep))
    return None if n < 0 else keep[:n].tolist()


def lse_merge(o: np.ndarray, lse: np.ndarray) -> np.ndarray:
    """o: [n_parts, D] normalised partial outputs, lse: [n_parts]. Returns merged [D]."""
    o = _f32(o)
    lse = _f32(lse)
    out = np.zeros(o.shape[1], dtype=np.float32)
    lib().orc_lse_merge(_p(o), _p(lse), o.shape[0], o.shape[1], _p(out))
    return out


# ── KV write and eviction executors (numpy restatements; test infrastructure like the rest of this file) ──

def kv_scatter(k_src, v_src, k_cache, v_cache, write_pos):
    """kv_scatter_f32_to_f16[_batch] / kv_scatter_f32_to_f32_batch (engine/src/backend/cuda_pc/kernels.cu:305-360):
    src [S, Hkv, D] F32 -> HeadMajor cache [Hkv, cap, D] rows write_pos.. (numpy's F32->F16 cast rounds to nearest even,
    as __float2half does). In place."""
    S = k_src.shape[0]
    with np.errstate(over="ignore"):   # values beyond the F16 range become inf, as on the device
        for s in range(S):
            k_cache[:, write_pos + s, :] = k_src[s].astype(k_cache.dtype)
            v_cache[:, write_pos + s, :] = v_src[s].astype(v_cache.dtype)


def compact_keep_positions(cache, keep, write_start, head=None):
    """KVCache::compact_keep_positions / _for_head (engine/src/kv/kv_cache.rs:1266-1352), literally: runs of consecutive
    source positions become one shift_positions call (a memmove of `count` rows), skipped when source == destination.
    cache [Hkv, cap, D], in place; head=None moves every head."""
    if len(keep) == 0:
        return
    heads = slice(None) if head is None else slice(head, head + 1)

    def shift(src, dst, count):
        cache[heads, dst:dst + count, :] = cache[heads, src:src + count, :].copy()

    write_pos = write_start
    batch_src, batch_dst, batch_count = keep[0], write_pos, 1
    write_pos += 1
    for src_pos in keep[1:]:
        if src_pos == batch_src + batch_count:
            batch_count += 1
        else:
            if batch_src != batch_dst:
                shift(batch_src, batch_dst, batch_count)
            batch_src, batch_dst, batch_count = src_pos, write_pos, 1
        write_pos += 1
    if batch_src != batch_dst:
        shift(batch_src, batch_dst, batch_count)


def apply_weighted_merges(k_cache, v_cache, merges, axis=0):
    """apply_weighted_merges, F32 and F16 arms (engine/src/kv/standard_format.rs:754-893): per merge (into, into_weight,
    [(from, w), ...]) and head, acc = into_w*x[into]; acc += w*x[from] in list order, products and sums rounded to F32
    one by one; an F16 cache converts on load and rounds once on store. axis 0 both, 1 K only, 2 V only. In place."""
    f32 = np.float32
    for into, into_w, frm in merges:
        if not frm:
            continue
        for buf, on in ((k_cache, axis != 2), (v_cache, axis != 1)):
            if not on:
                continue
            acc = f32(into_w) * buf[:, into, :].astype(f32)
            for pos, w in frm:
                acc = acc + f32(w) * buf[:, pos, :].astype(f32)
            buf[:, into, :] = acc.astype(buf.dtype)


def prefill_attention_scores(q, k, n_heads_kv, q_start_pos, q_window, cache_seq_len, window=None):
    """prefill_attention_scores (engine/src/kv/standard_format.rs:1400-1510), step by step as the reference: for each
    head h and each trailing row r (p = q_start_pos + r, keys lo..=p): scalar F32 dot in channel order, * 1/sqrt(D),
    max, exp(logit - max) with an F32 running denominator, prob = e / denom. q [S, Hq, D] F32, k [Hkv, cap, D] (any float
    dtype, read as F32). Returns (sum_out [Hq, prefix], per_row [qwin, Hq, prefix], head_mean [qwin, prefix])."""
    f32 = np.float32
    S, hq, d = q.shape
    g = hq // n_heads_kv
    prefix = cache_seq_len
    qwin = min(q_window, S)
    qwin_start = S - qwin
    scale = f32(1.0) / np.sqrt(f32(d))
    inv_heads = f32(1.0) / f32(hq)
    sum_out = np.zeros((hq, prefix), dtype=f32)
    per_row = np.zeros((qwin, hq, prefix), dtype=f32)
    head_mean = np.zeros((qwin, prefix), dtype=f32)
    kf = k.astype(f32)
    for h in range(hq):
        kvh = h // g
        for r in range(qwin_start, S):
            p = q_start_pos + r
            lo = 0 if window is None else max(0, p - max(window - 1, 0))
            keys = kf[kvh, lo:p + 1]                       # [n, D]
            dot = np.zeros(keys.shape[0], dtype=f32)
            for c in range(d):                              # the reference's channel-order scalar accumulation
                dot = dot + q[r, h, c] * keys[:, c]
            logit = dot * scale
            e = np.exp(logit - logit.max()).astype(f32)
            denom = f32(0.0)
            for x in e:                                     # sequential F32 sum
                denom = f32(denom + x)
            prob = (e / denom).astype(f32)
            sum_out[h, lo:p + 1] += prob
            per_row[r - qwin_start, h, lo:p + 1] = prob
            head_mean[r - qwin_start, lo:p + 1] += prob * inv_heads
    return sum_out, per_row, head_mean


def d2o_find_nearest(k_cache, evict_pos, retain_pos):
    """find_nearest_layer_wide_via + cosine_similarity (crates/techniques/d2o/src/lib.rs:187-255): k_cache [Hkv, cap, D];
    per evicted position the retained position of the largest cosine similarity between head-concatenated K rows
    (strict `>`: first in list order on ties; the evicted position itself is skipped; no valid target -> retain[0] or the
    evicted position, similarity 0). dot and the squared norms are accumulated channel by channel in F32, one rounding
    per product and per sum, exactly like the scalar loop. Returns (nearest int32 [E], sim float32 [E])."""
    f32 = np.float32
    hkv, _, d = k_cache.shape
    ev = np.asarray(evict_pos, dtype=np.int64)
    rt = np.asarray(retain_pos, dtype=np.int64)
    nearest = np.zeros(len(ev), dtype=np.int32)
    sims = np.zeros(len(ev), dtype=f32)
    if len(ev) == 0:
        return nearest, sims
    rows_e = k_cache[:, ev, :].astype(f32).transpose(1, 0, 2).reshape(len(ev), hkv * d)
    rows_r = k_cache[:, rt, :].astype(f32).transpose(1, 0, 2).reshape(len(rt), hkv * d) if len(rt) else np.zeros((0, hkv * d), f32)
    dot = np.zeros((len(ev), len(rt)), dtype=f32)
    na = np.zeros(len(ev), dtype=f32)
    nb = np.zeros(len(rt), dtype=f32)
    for c in range(hkv * d):
        a, b = rows_e[:, c], rows_r[:, c]
        dot = dot + a[:, None] * b[None, :]
        na = na + a * a
        nb = nb + b * b
    with np.errstate(divide="ignore", invalid="ignore"):
        denom = np.sqrt(na[:, None] * nb[None, :]).astype(f32)
        sim = np.where(denom < f32(1e-10), f32(0.0), (dot / denom).astype(f32)).astype(f32)
    for i, e in enumerate(ev):
        best_pos = int(rt[0]) if len(rt) else int(e)
        best = -np.inf
        for j, r in enumerate(rt):
            if r == e:
                continue
            if sim[i, j] > best:
                best, best_pos = sim[i, j], int(r)
        nearest[i] = best_pos
        sims[i] = f32(0.0) if best == -np.inf else best
    return nearest, sims


# ── session prefix cache file ("ARGUSKV1", version 2) ──

def extract_packed_bytes(cache: np.ndarray, token_count: int) -> bytes:
    """extract_packed_bytes for F32 / F16 caches (engine/src/kv/standard_format.rs:1657-1701): HeadMajor [Hkv, cap, D] ->
    the first token_count rows of every head, heads back to back."""
    return np.ascontiguousarray(cache[:, :token_count, :]).tobytes()


def prefix_cache_encode(model_hash: bytes, tokenizer_hash: bytes, token_ids, last_logits, format_id: int, kv_heads: int,
                        head_dim: int, layer_payloads) -> bytes:
    """save_prefix (engine/src/session/prefix_cache.rs:98-149): magic, version 2, header_len (fixed fields after it + the
    token ids), model hash, format id, tokenizer hash, geometry, token ids, logits section, then the layers' payloads
    (K bytes then V bytes each) in layer order. All integers little-endian u32, logits little-endian f32."""
    import struct

    assert len(model_hash) == 32 and len(tokenizer_hash) == 32
    token_ids = list(token_ids)
    header_len = (100 - 8 - 4 - 4) + 4 * len(token_ids)
    buf = bytearray(b"ARGUSKV1")
    buf += struct.pack("<II", 2, header_len)
    buf += model_hash
    buf += struct.pack("<I", format_id)
    buf += tokenizer_hash
    buf += struct.pack("<IIII", kv_heads, head_dim, len(layer_payloads), len(token_ids))
    buf += struct.pack(f"<{len(token_ids)}I", *token_ids)
    logits = np.asarray(last_logits, dtype="<f4")
    buf += struct.pack("<I", logits.size) + logits.tobytes()
    for payload in layer_payloads:
        buf += payload
    return bytes(buf)


def prefix_cache_decode(raw: bytes, n_layers: int):
    """The reading half of try_restore_prefix (engine/src/session/prefix_cache.rs:170-330) without the validation against
    a running model: returns the header fields and the payload split evenly over the layers, or None for a file the
    reference would invalidate by magic / version / truncation."""
    import struct

    if len(raw) < 100 or raw[:8] != b"ARGUSKV1":
        return None
    version, header_len = struct.unpack_from("<II", raw, 8)
    if version != 2:
        return None
    off = 16
    model_hash = raw[off:off + 32]
    off += 32
    (format_id,) = struct.unpack_from("<I", raw, off)
    off += 4
    tokenizer_hash = raw[off:off + 32]
    off += 32
    kv_heads, head_dim, saved_layers, token_count = struct.unpack_from("<IIII", raw, off)
    off += 16
    if saved_layers != n_layers or off + 4 * token_count > len(raw):
        return None
    token_ids = list(struct.unpack_from(f"<{token_count}I", raw, off))
    off += 4 * token_count
    (logits_len,) = struct.unpack_from("<I", raw, off)
    off += 4
    if off + 4 * logits_len > len(raw):
        return None
    logits = np.frombuffer(raw, dtype="<f4", count=logits_len, offset=off).copy()
    off += 4 * logits_len
    payload = raw[off:]
    if n_layers and len(payload) % n_layers:
        return None
    per = len(payload) // max(n_layers, 1)
    return {"model_hash": model_hash, "tokenizer_hash": tokenizer_hash, "format_id": format_id, "kv_heads": kv_heads,
            "head_dim": head_dim, "token_ids": token_ids, "last_logits": logits, "header_len": header_len,
            "layers": [payload[i * per:(i + 1) * per] for i in range(n_layers)]}
