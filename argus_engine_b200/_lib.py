"""ctypes binding of ``include/argus_b200.h`` (the same declarations a cgo/Rust FFI stub would carry)."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libargus_b200.so")


class ArgusB200Error(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"argus_b200 error {code}: {msg}")
        self.code = code


class PagedSeq(C.Structure):
    _fields_ = [("page_table", C.c_void_p), ("seq_len", C.c_int64)]


class Seq(C.Structure):
    _fields_ = [("k", C.c_void_p), ("v", C.c_void_p), ("seq_len", C.c_int64), ("head_stride", C.c_int64),
                ("pos_stride", C.c_int64)]


class DecodeExtrasC(C.Structure):
    _fields_ = [("scores", C.c_void_p), ("head_scores", C.c_void_p), ("flat_scores", C.c_void_p),
                ("lse", C.c_void_p), ("scores_host", C.c_void_p), ("score_stride", C.c_int64)]


class QuantAttnArgs(C.Structure):
    """CudaQuantAttnArgs (crates/argus-extension-api/src/lib.rs:3000-3026)."""
    _fields_ = [("cu_stream", C.c_void_p), ("q_mem", C.c_uint64), ("qk_mem", C.c_uint64), ("qv_mem", C.c_uint64),
                ("res_k_mem", C.c_uint64), ("res_v_mem", C.c_uint64), ("out_mem", C.c_uint64),
                ("scores_out", C.c_void_p), ("scores_len", C.c_size_t), ("num_heads_q", C.c_size_t),
                ("num_heads_kv", C.c_size_t), ("head_dim", C.c_size_t), ("q_tokens", C.c_size_t),
                ("res_tokens", C.c_size_t), ("res_cap", C.c_size_t), ("scale", C.c_float), ("bits", C.c_uint8)]


class QuantGatherArgs(C.Structure):
    _fields_ = [("cu_stream", C.c_void_p), ("input_mem", C.c_uint64), ("residual_mem", C.c_uint64),
                ("kv_heads", C.c_size_t), ("res_cap", C.c_size_t), ("head_dim", C.c_size_t), ("seq_len", C.c_size_t),
                ("res_pos", C.c_size_t)]


class QuantDequantFlushArgs(C.Structure):
    _fields_ = [("cu_stream", C.c_void_p), ("q_blocks_mem", C.c_uint64), ("attn_mem", C.c_uint64),
                ("kv_heads", C.c_size_t), ("head_dim", C.c_size_t), ("n_groups_or_tokens", C.c_size_t),
                ("tok_base", C.c_size_t), ("block_start", C.c_size_t), ("bits", C.c_uint8), ("is_key", C.c_uint8)]


class QuantScatterResidualArgs(C.Structure):
    _fields_ = [("cu_stream", C.c_void_p), ("res_mem", C.c_uint64), ("attn_mem", C.c_uint64),
                ("kv_heads", C.c_size_t), ("res_cap", C.c_size_t), ("head_dim", C.c_size_t), ("res_pos", C.c_size_t),
                ("tok_base", C.c_size_t)]


class KiviSeq(C.Structure):
    _fields_ = [("qk", C.c_void_p), ("qv", C.c_void_p), ("res_k", C.c_void_p), ("res_v", C.c_void_p),
                ("q_tokens", C.c_int64), ("res_tokens", C.c_int64)]


class KiviPagedSeq(C.Structure):
    _fields_ = [("flush_pages", C.c_void_p), ("res_k", C.c_void_p), ("res_v", C.c_void_p),
                ("q_tokens", C.c_int64), ("res_tokens", C.c_int64)]


class ExchangeC(C.Structure):
    """argus_b200_exchange."""
    _fields_ = [("peer_lines", C.POINTER(C.c_void_p)), ("step_counters", C.c_void_p), ("merged_lse", C.c_void_p),
                ("parity_stride_lines", C.c_int64), ("n_ranks", C.c_int), ("rank", C.c_int), ("phases", C.c_int)]


class ScoreReduceArgs(C.Structure):
    """CudaScoreReduceArgs (crates/argus-extension-api/src/lib.rs:2909-2933)."""
    _fields_ = [("cu_stream", C.c_void_p), ("score_buf", C.c_uint64), ("importance", C.c_uint64),
                ("head_importance", C.c_uint64), ("decay_factor", C.c_float), ("n_layers", C.c_size_t),
                ("n_heads_q", C.c_size_t), ("n_kv_heads", C.c_size_t), ("cache_seq_len", C.c_size_t),
                ("score_stride", C.c_size_t), ("max_seq_len", C.c_size_t), ("layer_flat_importance", C.c_uint64)]


_lib = None


def load_library() -> C.CDLL:
    """Load the CUDA library; fails loudly when it has not been built (no fallback exists)."""
    global _lib
    if _lib is not None:
        return _lib
    # ARGUS_B200_LIB_PATH selects another build of the same library (the time-stamped diagnostic twin, say).
    path = os.environ.get("ARGUS_B200_LIB_PATH") or LIB_PATH
    if not os.path.exists(path):
        raise ImportError(f"{path} is missing: run `python -m argus_engine_b200.build` "
                          "(or __graft_entry__.build()) first; there is no CPU fallback")
    lib = C.CDLL(path)
    vp, i32, i64 = C.c_void_p, C.c_int, C.c_int64
    lib.argus_b200_create.argtypes = [i32, C.c_size_t, C.POINTER(vp)]
    lib.argus_b200_create_in_context.argtypes = [vp, i32, C.c_size_t, C.POINTER(vp)]
    lib.argus_b200_destroy.argtypes = [vp]
    lib.argus_b200_destroy.restype = None
    lib.argus_b200_last_error.argtypes = [vp]
    lib.argus_b200_last_error.restype = C.c_char_p
    lib.argus_b200_launch_count.argtypes = [vp]
    lib.argus_b200_launch_count.restype = C.c_uint64
    lib.argus_b200_attention_gen.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, i64, i32, i64, i64,
                                             C.POINTER(DecodeExtrasC)]
    lib.argus_b200_attention_gen_batched.argtypes = [vp, vp, vp, C.POINTER(Seq), i32, vp, i32, i32, i32, i32,
                                                     C.POINTER(DecodeExtrasC)]
    lib.argus_b200_decode_step_batched.argtypes = [vp, vp, vp, vp, vp, C.POINTER(Seq), C.POINTER(i64), i32, vp, i32, i32, i32, i32,
                                                   C.POINTER(DecodeExtrasC)]
    lib.argus_b200_decode_step.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i64, i64, i32, i64, i64,
                                           C.POINTER(DecodeExtrasC)]
    lib.argus_b200_kivi_has_quant_attn_kernel.argtypes = [vp, i32]
    lib.argus_b200_kivi_attention_gen_quant.argtypes = [vp, C.POINTER(QuantAttnArgs)]
    lib.argus_b200_kivi_gather_update_quant.argtypes = [vp, C.POINTER(QuantGatherArgs)]
    lib.argus_b200_kivi_dequant_flush.argtypes = [vp, C.POINTER(QuantDequantFlushArgs)]
    lib.argus_b200_kivi_scatter_residual.argtypes = [vp, C.POINTER(QuantScatterResidualArgs)]
    lib.argus_b200_kivi_flush_pack.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i64, i64]
    lib.argus_b200_kivi_attention_batched.argtypes = [vp, vp, vp, C.POINTER(KiviSeq), i32, vp, i32, i32, i32, i32, i32,
                                                      i32, C.c_float, C.POINTER(DecodeExtrasC)]
    lib.argus_b200_kivi_attention_paged.argtypes = [vp, vp, vp, vp, vp, C.POINTER(KiviPagedSeq), i32, vp, i32, i32, i32,
                                                    i32, i32, i32, C.c_float, C.POINTER(DecodeExtrasC)]
    lib.argus_b200_score_reduce.argtypes = [vp, C.POINTER(ScoreReduceArgs)]
    lib.argus_b200_score_reduce_per_layer.argtypes = [vp, C.POINTER(ScoreReduceArgs)]
    lib.argus_b200_check_status.argtypes = [vp, vp]
    lib.argus_b200_flash_attention_prefill.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i64, i32, i32, i32]
    lib.argus_b200_lse_merge.argtypes = [vp, vp, vp, i32, i64, i32, i32, vp, vp]
    lib.argus_b200_exchange_wait_merge.argtypes = [vp, vp, vp, C.POINTER(ExchangeC), i32, i32, i32, i32, vp]
    lib.argus_b200_exchange_lines_per_head.argtypes = [i32, i32, i32]
    lib.argus_b200_attention_gen_sharded.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, i64, i32, i64, i64,
                                                     C.POINTER(ExchangeC)]
    lib.argus_b200_kv_scatter.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, i64, i64, i64, i64, i64]
    lib.argus_b200_prefill_attention_scores.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i64, i64, i32, i32, i32,
                                                        vp, vp, i32]
    lib.argus_b200_kv_scatter_batched.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32]
    lib.argus_b200_d2o_nearest.argtypes = [vp, vp, vp, i32, i32, i32, i64, i64, vp, i32, vp, i32, vp, vp]
    lib.argus_b200_attention_gen_paged.argtypes = [vp, vp, vp, vp, vp, vp, i32, vp, i32, i32, i32, i32, i64, i64, i64, vp]
    lib.argus_b200_kv_compact.argtypes = [vp, vp, vp, vp, i32, i32, i32, i64, i64, i64, vp, i64, i64, i32]
    lib.argus_b200_kv_weighted_merge.argtypes = [vp, vp, vp, vp, i32, i32, i32, i64, i64, vp, vp, vp, vp, vp, i32, i32]
    lib.argus_b200_kv_snapshot_prefix.argtypes = [vp, vp, vp, vp, i32, i32, i32, i64, i64, i64, i64, vp, C.c_size_t]
    lib.argus_b200_kv_restore_prefix.argtypes = [vp, vp, vp, vp, i32, i32, i32, i64, i64, i64, i64, vp, C.c_size_t]
    lib.argus_b200_kv_make_resident.argtypes = [vp, vp, vp, C.c_size_t]
    lib.argus_b200_kv_alloc.argtypes = [vp, C.c_size_t, i32, C.POINTER(vp)]
    lib.argus_b200_kv_free.argtypes = [vp, vp]
    lib.argus_b200_attention_gen_static.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, i64, i32, i64, i64]
    lib.argus_b200_static_scratch_bytes.restype = C.c_size_t
    lib.argus_b200_static_last_error.restype = C.c_char_p
    _lib = lib
    return lib
