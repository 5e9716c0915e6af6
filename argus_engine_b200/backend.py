"""Host-side mirror of the reference's attention entry points over the C ABI.

Method names, argument order and error behaviour follow ``trait Backend`` of the reference
(engine/src/backend.rs:284-295 ``attention_gen``, :1011-1027 ``flash_attention_prefill``), so the parity
tests read like the reference's own. torch is used only as the owner of device memory and streams.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from ._lib import (ArgusB200Error, DecodeExtrasC, ExchangeC, KiviPagedSeq, KiviSeq, QuantAttnArgs, QuantDequantFlushArgs,
                   QuantGatherArgs, QuantScatterResidualArgs, PagedSeq, ScoreReduceArgs, Seq, load_library)

KV_F32, KV_F16 = 0, 1


@dataclass
class DecodeExtras:
    """Optional outputs of a decode call (see ``argus_b200_decode_extras`` in the C header)."""
    scores: Optional[torch.Tensor] = None        # [B, Hq, stride] f32 device
    head_scores: Optional[torch.Tensor] = None   # [B, Hkv, stride] f32 device
    flat_scores: Optional[torch.Tensor] = None   # [B, stride] f32 device
    lse: Optional[torch.Tensor] = None           # [B, Hq] f32 device
    scores_host: Optional[torch.Tensor] = None   # [B, Hq, stride] f32 host (blocking read-back)
    score_stride: int = 0


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


class B200Backend:
    """One per device; owns the library context (split-KV scratch)."""

    def __init__(self, device: int = 0, workspace_bytes: int = 0, cu_context: Optional[int] = None):
        """cu_context: a raw CUcontext to create the library context in (argus_b200_create_in_context, the route the
        engine's plugin factory takes); None binds the device's primary context."""
        self._lib = load_library()
        if not torch.cuda.is_available():
            raise RuntimeError("argus_engine_b200 needs a CUDA device (there is no CPU fallback)")
        torch.cuda.set_device(device)
        torch.cuda.init()
        h = C.c_void_p()
        if cu_context is not None:
            rc = self._lib.argus_b200_create_in_context(C.c_void_p(cu_context), device, workspace_bytes, C.byref(h))
        else:
            rc = self._lib.argus_b200_create(device, workspace_bytes, C.byref(h))
        if rc != 0:
            raise ArgusB200Error(rc, "argus_b200_create failed (is this an sm_100 device?)")
        self._h = h
        self.device = device

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.argus_b200_destroy(self._h)
            self._h = None

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass

    # ── helpers ──
    def _check(self, rc: int) -> None:
        if rc != 0:
            raise ArgusB200Error(rc, self._lib.argus_b200_last_error(self._h).decode())

    @property
    def launch_count(self) -> int:
        return int(self._lib.argus_b200_launch_count(self._h))

    @staticmethod
    def _stream() -> int:
        return torch.cuda.current_stream().cuda_stream

    @staticmethod
    def _extras(ex: Optional[DecodeExtras]):
        if ex is None:
            return None
        c = DecodeExtrasC(_ptr(ex.scores), _ptr(ex.head_scores), _ptr(ex.flat_scores), _ptr(ex.lse),
                          _ptr(ex.scores_host), int(ex.score_stride))
        return C.byref(c)

    @staticmethod
    def kv_strides(k_cache: torch.Tensor, num_heads_kv: int):
        """(head_stride, pos_stride, is_head_major) by the reference's shape rule
        (engine/src/backend.rs:336-339): HeadMajor iff rank>=3, shape[-3]==Hkv and shape[-3]!=shape[-2]."""
        shp = k_cache.shape
        if k_cache.stride(-1) != 1:
            raise ValueError("the channel dimension of a KV cache must be contiguous")
        # strides come from the tensor, so that a view of a larger cache (a slice of positions) is addressed correctly
        if len(shp) >= 3 and shp[-3] == num_heads_kv and shp[-3] != shp[-2]:
            return k_cache.stride(-3), k_cache.stride(-2), True
        if len(shp) >= 3:
            return k_cache.stride(-2), k_cache.stride(-3), False
        return shp[-1], num_heads_kv * shp[-1], False

    # ── Backend::attention_gen ──
    def attention_gen(self, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                      num_heads_q: int, num_heads_kv: int, head_dim: int, cache_seq_len: int,
                      scores_out: Optional[torch.Tensor] = None, extras: Optional[DecodeExtras] = None) -> None:
        """q [Hq,D] f32; K/V f16 HeadMajor [Hkv,cap,D] or SeqMajor [T,Hkv,D]; out [Hq,D] f32.
        ``scores_out``: optional [Hq, stride] tensor (device, or host for the blocking read-back form)."""
        hs, ps, _ = self.kv_strides(k_cache, num_heads_kv)
        if scores_out is not None:
            extras = extras or DecodeExtras()
            extras.score_stride = scores_out.numel() // num_heads_q
            if scores_out.is_cuda:
                extras.scores = scores_out
            else:
                extras.scores_host = scores_out
        dt = KV_F16 if k_cache.dtype == torch.float16 else KV_F32
        self._check(self._lib.argus_b200_attention_gen(
            self._h, self._stream(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
            num_heads_q, num_heads_kv, head_dim, cache_seq_len, dt, hs, ps, self._extras(extras)))

    def attention_gen_batched(self, q: torch.Tensor, k_caches: Sequence[torch.Tensor],
                              v_caches: Sequence[torch.Tensor], seq_lens: Sequence[int], out: torch.Tensor,
                              num_heads_q: int, num_heads_kv: int, head_dim: int,
                              extras: Optional[DecodeExtras] = None) -> None:
        """Independent sequences of different lengths in one launch. q/out [B,Hq,D]."""
        n = len(k_caches)
        arr = (Seq * n)()
        for i in range(n):
            hs, ps, _ = self.kv_strides(k_caches[i], num_heads_kv)
            arr[i] = Seq(k_caches[i].data_ptr(), v_caches[i].data_ptr(), int(seq_lens[i]), hs, ps)
        dt = KV_F16 if k_caches[0].dtype == torch.float16 else KV_F32
        self._check(self._lib.argus_b200_attention_gen_batched(
            self._h, self._stream(), q.data_ptr(), arr, n, out.data_ptr(), num_heads_q, num_heads_kv, head_dim, dt,
            self._extras(extras)))

    def decode_step_batched(self, q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, k_caches, v_caches, write_pos,
                            out: torch.Tensor, num_heads_q: int, num_heads_kv: int, head_dim: int,
                            extras: Optional[DecodeExtras] = None) -> None:
        """KV write + attention of one decode step in one call. k_new/v_new [B, Hkv, D] F32 are stored at position
        write_pos[b] (the sequence's length before the step) of cache b [Hkv, cap, D]; the attention covers
        write_pos[b] + 1 positions. q/out [B, Hq, D]."""
        n = len(k_caches)
        arr = (Seq * n)()
        cap = (C.c_int64 * n)()
        for i in range(n):
            hs, ps, _ = self.kv_strides(k_caches[i], num_heads_kv)
            arr[i] = Seq(k_caches[i].data_ptr(), v_caches[i].data_ptr(), int(write_pos[i]), hs, ps)
            cap[i] = k_caches[i].shape[-2] if k_caches[i].dim() >= 3 and k_caches[i].shape[-3] == num_heads_kv else k_caches[i].shape[0]
        dt = KV_F16 if k_caches[0].dtype == torch.float16 else KV_F32
        self._check(self._lib.argus_b200_decode_step_batched(
            self._h, self._stream(), q.data_ptr(), k_new.data_ptr(), v_new.data_ptr(), arr, cap, n, out.data_ptr(), num_heads_q,
            num_heads_kv, head_dim, dt, self._extras(extras)))

    def decode_step(self, q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, k_cache: torch.Tensor,
                    v_cache: torch.Tensor, out: torch.Tensor, num_heads_q: int, num_heads_kv: int, head_dim: int,
                    cache_seq_len: int, extras: Optional[DecodeExtras] = None) -> None:
        """Single-sequence form: k_new/v_new [Hkv, D] F32 written at position cache_seq_len, attention over cache_seq_len+1."""
        self.decode_step_batched(q, k_new, v_new, [k_cache], [v_cache], [cache_seq_len], out, num_heads_q, num_heads_kv,
                                 head_dim, extras)

    def attention_gen_paged(self, q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, page_tables, seq_lens,
                            out: torch.Tensor, num_heads_q: int, extras: Optional[DecodeExtras] = None) -> None:
        """Batched decode over paged F16 caches. Pools [n_pages, Hkv, page_tokens, D]; page_tables: one int32 device
        tensor per sequence; q/out [B, Hq, D]."""
        n_pages, hkv, ptok, d = k_pool.shape
        n = len(page_tables)
        arr = (PagedSeq * n)()
        for i in range(n):
            arr[i] = PagedSeq(page_tables[i].data_ptr() if page_tables[i] is not None else None, int(seq_lens[i]))
        self._check(self._lib.argus_b200_attention_gen_paged(
            self._h, self._stream(), q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), arr, n, out.data_ptr(), num_heads_q,
            hkv, d, ptok, k_pool.stride(0), k_pool.stride(1), k_pool.stride(2), self._extras(extras)))

    # ── Backend::flash_attention_prefill ──
    def flash_attention_prefill(self, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                                n_heads_q: int, n_heads_kv: int, seq_len: int, cache_seq_len: int, head_dim: int,
                                kv_capacity: int, batch_size: int, is_head_major: bool) -> bool:
        """Argument list of the reference trait method (engine/src/backend.rs:1011-1027). Returns True when the
        GPU kernel handled the call, False when it declines (the reference's ``Ok(false)``); errors raise.
        dtype mode follows the tensors: F32 Q + F16 K/V + F32 out (the engine's), all-BF16, or all-F16."""
        if q.dtype == torch.float32 and k_cache.dtype == torch.float16 and out.dtype == torch.float32:
            mode = 0
        elif q.dtype == k_cache.dtype == out.dtype == torch.bfloat16:
            mode = 1
        elif q.dtype == k_cache.dtype == out.dtype == torch.float16:
            mode = 2
        else:
            return False
        rc = self._lib.argus_b200_flash_attention_prefill(
            self._h, self._stream(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), n_heads_q,
            n_heads_kv, seq_len, cache_seq_len, head_dim, kv_capacity, batch_size, int(bool(is_head_major)), mode)
        if rc == -2:
            return False
        self._check(rc)
        return True

    # ── CudaQuantAttnBackend (crates/argus-extension-api/src/lib.rs:3087-3104) ──
    def has_quant_attn_kernel(self, bits: int) -> bool:
        return bool(self._lib.argus_b200_kivi_has_quant_attn_kernel(self._h, bits))

    def attention_gen_quant(self, q, qk, qv, res_k, res_v, out, num_heads_q, num_heads_kv, head_dim, q_tokens,
                            res_tokens, res_cap, scale, bits, scores_out: Optional[torch.Tensor] = None) -> int:
        """Argument meaning of CudaQuantAttnArgs; ``scores_out`` is a HOST tensor [Hq, stride] or None.
        Returns the reference's status code (0 ok, negative on failure) instead of raising."""
        a = QuantAttnArgs(self._stream(), q.data_ptr(), _ptr(qk) or 0, _ptr(qv) or 0, _ptr(res_k) or 0, _ptr(res_v) or 0,
                          out.data_ptr(), _ptr(scores_out), 0 if scores_out is None else scores_out.numel(),
                          num_heads_q, num_heads_kv, head_dim, q_tokens, res_tokens, res_cap, float(scale), bits)
        return int(self._lib.argus_b200_kivi_attention_gen_quant(self._h, C.byref(a)))

    def gather_update_quant(self, inp, residual, kv_heads, res_cap, head_dim, seq_len, res_pos) -> int:
        a = QuantGatherArgs(self._stream(), inp.data_ptr(), residual.data_ptr(), kv_heads, res_cap, head_dim, seq_len,
                            res_pos)
        return int(self._lib.argus_b200_kivi_gather_update_quant(self._h, C.byref(a)))

    def dequant_flush(self, q_blocks, attn, kv_heads, head_dim, n_groups_or_tokens, tok_base, block_start, bits,
                      is_key) -> int:
        a = QuantDequantFlushArgs(self._stream(), q_blocks.data_ptr(), attn.data_ptr(), kv_heads, head_dim,
                                  n_groups_or_tokens, tok_base, block_start, bits, int(bool(is_key)))
        return int(self._lib.argus_b200_kivi_dequant_flush(self._h, C.byref(a)))

    def scatter_residual(self, res, attn, kv_heads, res_cap, head_dim, res_pos, tok_base) -> int:
        a = QuantScatterResidualArgs(self._stream(), res.data_ptr(), attn.data_ptr(), kv_heads, res_cap, head_dim,
                                     res_pos, tok_base)
        return int(self._lib.argus_b200_kivi_scatter_residual(self._h, C.byref(a)))

    def kivi_flush_pack(self, res_k, res_v, qk, qv, kv_heads, head_dim, res_cap, n_groups, bits, k_block_start,
                        v_block_start) -> None:
        """Device-side flush of the residual ring into packed blocks (bit-exact with the CPU codec)."""
        self._check(self._lib.argus_b200_kivi_flush_pack(self._h, self._stream(), res_k.data_ptr(), res_v.data_ptr(),
                                                         qk.data_ptr(), qv.data_ptr(), kv_heads, head_dim, res_cap,
                                                         n_groups, bits, k_block_start, v_block_start))

    def kivi_attention_batched(self, q, seqs, out, num_heads_q, num_heads_kv, head_dim, res_cap, bits, scale,
                               res_f16: bool = False, extras: Optional[DecodeExtras] = None) -> None:
        """seqs: list of (qk, qv, res_k, res_v, q_tokens, res_tokens) with device tensors (or None when empty)."""
        n = len(seqs)
        arr = (KiviSeq * n)()
        for i, (qk, qv, rk, rv, qt, rt) in enumerate(seqs):
            arr[i] = KiviSeq(_ptr(qk), _ptr(qv), _ptr(rk), _ptr(rv), int(qt), int(rt))
        self._check(self._lib.argus_b200_kivi_attention_batched(
            self._h, self._stream(), q.data_ptr(), arr, n, out.data_ptr(), num_heads_q, num_heads_kv, head_dim, res_cap,
            bits, KV_F16 if res_f16 else KV_F32, float(scale), self._extras(extras)))

    def kivi_attention_paged(self, q, qk_pool, qv_pool, seqs, out, num_heads_q, num_heads_kv, head_dim, res_cap, bits,
                             scale, res_f16: bool = False, extras: Optional[DecodeExtras] = None) -> None:
        """seqs: list of (flush_pages int32 device tensor, res_k, res_v, q_tokens, res_tokens); a page of the two pools
        holds one flush of res_cap tokens for all KV heads."""
        n = len(seqs)
        arr = (KiviPagedSeq * n)()
        for i, (pages, rk, rv, qt, rt) in enumerate(seqs):
            arr[i] = KiviPagedSeq(_ptr(pages), _ptr(rk), _ptr(rv), int(qt), int(rt))
        self._check(self._lib.argus_b200_kivi_attention_paged(
            self._h, self._stream(), q.data_ptr(), qk_pool.data_ptr(), qv_pool.data_ptr(), arr, n, out.data_ptr(),
            num_heads_q, num_heads_kv, head_dim, res_cap, bits, KV_F16 if res_f16 else KV_F32, float(scale),
            self._extras(extras)))

    # ── CudaScoreReduceBackend (crates/argus-extension-api/src/lib.rs:2938-2948) ──
    def _reduce_args(self, score_buf, importance, head_importance, decay_factor, n_layers, n_heads_q, n_kv_heads,
                     cache_seq_len, score_stride, max_seq_len, layer_flat):
        return ScoreReduceArgs(self._stream(), score_buf.data_ptr(), _ptr(importance) or 0, _ptr(head_importance) or 0,
                               float(decay_factor), n_layers, n_heads_q, n_kv_heads, cache_seq_len, score_stride,
                               max_seq_len, _ptr(layer_flat) or 0)

    def score_reduce(self, score_buf, importance, head_importance, decay_factor, n_layers, n_heads_q, n_kv_heads,
                     cache_seq_len, score_stride, max_seq_len, layer_flat=None) -> int:
        a = self._reduce_args(score_buf, importance, head_importance, decay_factor, n_layers, n_heads_q, n_kv_heads,
                              cache_seq_len, score_stride, max_seq_len, layer_flat)
        return int(self._lib.argus_b200_score_reduce(self._h, C.byref(a)))

    def score_reduce_per_layer(self, score_buf, layer_flat, decay_factor, n_layers, n_heads_q, n_kv_heads,
                               cache_seq_len, score_stride, max_seq_len) -> int:
        a = self._reduce_args(score_buf, None, None, decay_factor, n_layers, n_heads_q, n_kv_heads, cache_seq_len,
                              score_stride, max_seq_len, layer_flat)
        return int(self._lib.argus_b200_score_reduce_per_layer(self._h, C.byref(a)))

    def lse_merge(self, parts: torch.Tensor, num_heads_q: int, head_dim: int, out: torch.Tensor,
                  lse_out: Optional[torch.Tensor] = None) -> None:
        """parts [n_parts, Hq*D + Hq] f32 (per rank: outputs then lse) -> out [Hq, D]."""
        self._check(self._lib.argus_b200_lse_merge(self._h, self._stream(), parts.data_ptr(), parts.shape[0],
                                                   parts.stride(0), num_heads_q, head_dim, out.data_ptr(),
                                                   _ptr(lse_out)))

    def exchange_lines_per_head(self, num_heads_q: int, num_heads_kv: int, head_dim: int) -> int:
        return int(self._lib.argus_b200_exchange_lines_per_head(num_heads_q, num_heads_kv, head_dim))

    def _exchange(self, peer_lines, rank, step_counters, parity_stride_lines, merged_lse, phases):
        n = len(peer_lines)
        pl = (C.c_void_p * n)(*peer_lines)
        xc = ExchangeC(pl, _ptr(step_counters), _ptr(merged_lse), parity_stride_lines, n, rank, phases)
        xc._keep = pl
        return xc

    def attention_gen_sharded(self, q: torch.Tensor, k_shard: torch.Tensor, v_shard: torch.Tensor, out: torch.Tensor,
                              num_heads_q: int, num_heads_kv: int, head_dim: int, shard_len: int, peer_lines, rank: int,
                              step_counters: torch.Tensor, parity_stride_lines: int,
                              merged_lse: Optional[torch.Tensor] = None, phases: int = 3) -> None:
        """One launch per step of a sequence-sharded decode: split-KV decode over this rank's K/V slice whose epilogue
        pushes the (o, lse) rows to every rank and merges. peer_lines: device addresses (ints) of every rank's receive
        buffer; step_counters: int32 device tensor [Hkv], zero before the first step."""
        xc = self._exchange(peer_lines, rank, step_counters, parity_stride_lines, merged_lse, phases)
        hs, ps, _ = self.kv_strides(k_shard, num_heads_kv)
        dt = KV_F16 if k_shard.dtype == torch.float16 else KV_F32
        self._check(self._lib.argus_b200_attention_gen_sharded(
            self._h, self._stream(), q.data_ptr(), k_shard.data_ptr(), v_shard.data_ptr(), out.data_ptr(), num_heads_q,
            num_heads_kv, head_dim, shard_len, dt, hs, ps, C.byref(xc)))

    def exchange_wait_merge(self, own_part: torch.Tensor, peer_lines, rank: int, step: int, parity_stride_lines: int,
                            num_heads_q: int, num_heads_kv: int, head_dim: int, out: torch.Tensor,
                            merged_lse: Optional[torch.Tensor] = None) -> None:
        """The receiving half of the exchange as a launch of its own (after attention_gen_sharded with phases=1)."""
        xc = self._exchange(peer_lines, rank, None, parity_stride_lines, merged_lse, 2)
        self._check(self._lib.argus_b200_exchange_wait_merge(self._h, self._stream(), own_part.data_ptr(), C.byref(xc), step,
                                                             num_heads_q, num_heads_kv, head_dim, out.data_ptr()))

    # ── KV write and eviction executors (HeadMajor [Hkv, cap, D] caches, F16 or F32) ──
    @staticmethod
    def _kv_layout(k_cache: torch.Tensor):
        if k_cache.dim() != 3 or k_cache.stride(2) != 1 or k_cache.dtype not in (torch.float16, torch.float32):
            raise ValueError("expected a [Hkv, cap, D] F16/F32 cache with contiguous rows")
        return 1 if k_cache.dtype == torch.float16 else 0, k_cache.stride(0), k_cache.stride(1)

    def kv_scatter(self, k_src: torch.Tensor, v_src: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                   write_pos: int) -> None:
        """kv_scatter_f32_to_f16[_batch] / f32_to_f32_batch: rows k_src/v_src [S, Hkv, D] F32 -> cache positions
        write_pos .. write_pos+S-1."""
        dt, hs, ps = self._kv_layout(k_cache)
        S, hkv, d = k_src.shape
        self._check(self._lib.argus_b200_kv_scatter(self._h, self._stream(), k_src.data_ptr(), v_src.data_ptr(),
                                                    k_cache.data_ptr(), v_cache.data_ptr(), dt, hkv, d, k_cache.shape[1],
                                                    hs, ps, write_pos, S))

    def kv_scatter_batched(self, k_src: torch.Tensor, v_src: torch.Tensor, k_caches, v_caches, write_pos) -> None:
        """One new row per sequence in one launch: k_src/v_src [B, Hkv, D] F32 -> cache b at position write_pos[b]."""
        n = len(k_caches)
        B, hkv, d = k_src.shape
        arr = (Seq * n)()
        cap = (C.c_int64 * n)()
        for i in range(n):
            dt, hs, ps = self._kv_layout(k_caches[i])
            arr[i] = Seq(k_caches[i].data_ptr(), v_caches[i].data_ptr(), int(write_pos[i]), hs, ps)
            cap[i] = k_caches[i].shape[1]
        self._check(self._lib.argus_b200_kv_scatter_batched(self._h, self._stream(), k_src.data_ptr(), v_src.data_ptr(), arr,
                                                            cap, n, dt, hkv, d))

    def kv_compact(self, k_cache: torch.Tensor, v_cache: torch.Tensor, keep: torch.Tensor, write_start: int,
                   head: int = -1) -> None:
        """KVCache::compact_keep_positions (head = -1) / _for_head: position write_start+i <- position keep[i], in place.
        keep: ascending int32 device tensor."""
        dt, hs, ps = self._kv_layout(k_cache)
        if keep.dtype != torch.int32 or not keep.is_cuda:
            raise ValueError("keep must be an int32 device tensor")
        self._check(self._lib.argus_b200_kv_compact(self._h, self._stream(), k_cache.data_ptr(), v_cache.data_ptr(), dt,
                                                    k_cache.shape[0], k_cache.shape[2], k_cache.shape[1], hs, ps,
                                                    keep.data_ptr(), keep.numel(), write_start, head))

    def kv_weighted_merge(self, k_cache: torch.Tensor, v_cache: torch.Tensor, into_pos: torch.Tensor,
                          into_weight: torch.Tensor, from_start: torch.Tensor, from_pos: torch.Tensor,
                          from_weight: torch.Tensor, axis: int = 0) -> None:
        """apply_weighted_merges (F32/F16 arms): CSR lists on the device, axis 0 both / 1 K only / 2 V only."""
        dt, hs, ps = self._kv_layout(k_cache)
        self._check(self._lib.argus_b200_kv_weighted_merge(
            self._h, self._stream(), k_cache.data_ptr(), v_cache.data_ptr(), dt, k_cache.shape[0], k_cache.shape[2], hs,
            ps, into_pos.data_ptr(), into_weight.data_ptr(), from_start.data_ptr(), from_pos.data_ptr(),
            from_weight.data_ptr(), into_pos.numel(), axis))

    def d2o_nearest(self, k_cache: torch.Tensor, evict_pos: torch.Tensor, retain_pos: torch.Tensor):
        """find_nearest_layer_wide_via for every evicted position: (nearest retained position int32 [E], similarity f32 [E])."""
        dt, hs, ps = self._kv_layout(k_cache)
        n_e, n_r = evict_pos.numel(), retain_pos.numel()
        nearest = torch.empty(n_e, dtype=torch.int32, device=k_cache.device)
        sim = torch.empty(n_e, dtype=torch.float32, device=k_cache.device)
        self._check(self._lib.argus_b200_d2o_nearest(self._h, self._stream(), k_cache.data_ptr(), dt, k_cache.shape[0],
                                                     k_cache.shape[2], hs, ps, _ptr(evict_pos) if n_e else None, n_e,
                                                     _ptr(retain_pos) if n_r else None, n_r, nearest.data_ptr(), sim.data_ptr()))
        return nearest, sim

    def prefill_attention_scores(self, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, cache_seq_len: int,
                                 q_start_pos: int, q_window: int, sum_out: Optional[torch.Tensor] = None,
                                 per_row: Optional[torch.Tensor] = None, per_row_per_head: bool = True,
                                 window: int = 0) -> None:
        """prefill_attention_scores: q [S, Hq, D] F32, caches HeadMajor [Hkv, cap, D] F16; sum_out [Hq, cache_seq_len],
        per_row [q_window, Hq, cache_seq_len] (per head) or [q_window, cache_seq_len] (head mean), pre-zeroed."""
        dt, hs, ps = self._kv_layout(k_cache)
        S, hq, d = q.shape
        self._check(self._lib.argus_b200_prefill_attention_scores(
            self._h, self._stream(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), dt, hq, k_cache.shape[0], d, S,
            cache_seq_len, hs, ps, q_start_pos, q_window, window, _ptr(sum_out), _ptr(per_row), int(per_row_per_head)))

    def _prefix_layout(self, k_cache: torch.Tensor, num_heads_kv: int):
        hs, ps, head_major = self.kv_strides(k_cache, num_heads_kv)
        d = k_cache.shape[-1]
        cap = k_cache.shape[-2] if head_major else k_cache.shape[-3]
        dt = KV_F16 if k_cache.dtype == torch.float16 else KV_F32
        return dt, d, cap, hs, ps

    def kv_snapshot_prefix(self, k_cache: torch.Tensor, v_cache: torch.Tensor, num_heads_kv: int, token_count: int,
                           dst: torch.Tensor) -> None:
        """SnapshotRestore::snapshot_prefix payload of one layer: K bytes [Hkv, token_count, D] then V bytes into `dst`
        (a uint8 tensor of exactly that size, on the device or in pinned host memory)."""
        dt, d, cap, hs, ps = self._prefix_layout(k_cache, num_heads_kv)
        self._check(self._lib.argus_b200_kv_snapshot_prefix(self._h, self._stream(), k_cache.data_ptr(), v_cache.data_ptr(), dt,
                                                            num_heads_kv, d, cap, hs, ps, token_count, dst.data_ptr(),
                                                            dst.numel() * dst.element_size()))

    def kv_restore_prefix(self, k_cache: torch.Tensor, v_cache: torch.Tensor, num_heads_kv: int, token_count: int,
                          src: torch.Tensor) -> None:
        """SnapshotRestore::restore_prefix: the inverse of kv_snapshot_prefix into a cache of any capacity >= token_count."""
        dt, d, cap, hs, ps = self._prefix_layout(k_cache, num_heads_kv)
        self._check(self._lib.argus_b200_kv_restore_prefix(self._h, self._stream(), k_cache.data_ptr(), v_cache.data_ptr(), dt,
                                                           num_heads_kv, d, cap, hs, ps, token_count, src.data_ptr(),
                                                           src.numel() * src.element_size()))

    def kv_alloc(self, nbytes: int, managed: bool) -> int:
        """Raw KV allocation (managed = what the engine's CUDA backend uses). Returns the address."""
        out = C.c_void_p()
        self._check(self._lib.argus_b200_kv_alloc(self._h, nbytes, int(managed), C.byref(out)))
        return int(out.value)

    def kv_free(self, ptr: int) -> None:
        self._check(self._lib.argus_b200_kv_free(self._h, C.c_void_p(ptr)))

    def kv_make_resident(self, ptr: int, nbytes: int) -> None:
        """Preferred location = this device + prefetch, for a managed KV buffer (no-op for device memory)."""
        self._check(self._lib.argus_b200_kv_make_resident(self._h, self._stream(), C.c_void_p(ptr), nbytes))

    def check_status(self) -> int:
        """Synchronises the current stream; non-zero if a kernel's bounded wait ran out since the last check."""
        return int(self._lib.argus_b200_check_status(self._h, self._stream()))
