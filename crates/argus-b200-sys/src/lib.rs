//! FFI declarations for `include/argus_b200.h` and the trait glue that registers the B200 kernels behind
//! argus-engine's own plugin surface. The `#[repr(C)]` argument structs of `argus-extension-api` are passed
//! through unchanged: the C header declares byte-identical PODs (checked there with `static_assert`, here with
//! the `const` assertions at the bottom).

use std::ffi::{c_char, c_int, c_void, CStr};

use argus_extension_api::{
    CudaQuantAttnArgs, CudaQuantAttnBackend, CudaQuantAttnGatherArgs, CudaQuantAttnMakeArgs, CudaQuantAttnReg,
    CudaQuantDequantFlushArgs, CudaQuantScatterResidualArgs, CudaScoreReduceArgs, CudaScoreReduceBackend,
    CudaScoreReduceMakeArgs, CudaScoreReduceReg, CUDA_QUANT_ATTN_REGS, CUDA_SCORE_REDUCERS,
};
use linkme::distributed_slice;

/// `argus_b200_seq`: one sequence of a batched call (strides in elements).
#[repr(C)]
pub struct ArgusB200Seq {
    pub k: *const c_void,
    pub v: *const c_void,
    pub seq_len: i64,
    pub head_stride: i64,
    pub pos_stride: i64,
}

/// `argus_b200_paged_seq`: one sequence of a paged decode call.
#[repr(C)]
pub struct ArgusB200PagedSeq {
    pub page_table: *const i32,
    pub seq_len: i64,
}

#[repr(C)]
pub struct ArgusB200Ctx {
    _private: [u8; 0],
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct ArgusB200DecodeExtras {
    pub scores: *mut f32,
    pub head_scores: *mut f32,
    pub flat_scores: *mut f32,
    pub lse: *mut f32,
    pub scores_host: *mut f32,
    pub score_stride: i64,
}

/// `argus_b200_kivi_seq`: one KIVI-packed sequence of a batched call.
#[repr(C)]
pub struct ArgusB200KiviSeq {
    pub qk: *const c_void,
    pub qv: *const c_void,
    pub res_k: *const c_void,
    pub res_v: *const c_void,
    pub q_tokens: i64,
    pub res_tokens: i64,
}

/// `argus_b200_kivi_paged_seq`: one sequence of a paged KIVI call (a page = one flush of all KV heads).
#[repr(C)]
pub struct ArgusB200KiviPagedSeq {
    pub flush_pages: *const i32,
    pub res_k: *const c_void,
    pub res_v: *const c_void,
    pub q_tokens: i64,
    pub res_tokens: i64,
}

/// `argus_b200_exchange`: peer buffers of a sequence-sharded decode step.
#[repr(C)]
pub struct ArgusB200Exchange {
    pub peer_lines: *const *mut c_void,
    pub step_counters: *mut c_int,
    pub merged_lse: *mut f32,
    pub parity_stride_lines: i64,
    pub n_ranks: c_int,
    pub rank: c_int,
    pub phases: c_int,
}

pub const ARGUS_B200_KV_F32: c_int = 0;
pub const ARGUS_B200_KV_F16: c_int = 1;
pub const ARGUS_B200_E_UNSUPPORTED: c_int = -2;

extern "C" {
    pub fn argus_b200_create(device: c_int, workspace_bytes: usize, out: *mut *mut ArgusB200Ctx) -> c_int;
    pub fn argus_b200_create_in_context(
        cu_context: *mut c_void, device: c_int, workspace_bytes: usize, out: *mut *mut ArgusB200Ctx,
    ) -> c_int;
    pub fn argus_b200_destroy(ctx: *mut ArgusB200Ctx);
    pub fn argus_b200_version() -> c_int;
    pub fn argus_b200_sm_arch() -> c_int;
    pub fn argus_b200_launch_count(ctx: *const ArgusB200Ctx) -> u64;
    pub fn argus_b200_check_status(ctx: *mut ArgusB200Ctx, stream: *mut c_void) -> c_int;
    pub fn argus_b200_attention_gen_batched(
        ctx: *mut ArgusB200Ctx, stream: *mut c_void, q: *const f32, seqs: *const ArgusB200Seq, n_seqs: c_int,
        out: *mut f32, num_heads_q: c_int, num_heads_kv: c_int, head_dim: c_int, kv_dtype: c_int,
        extras: *const ArgusB200DecodeExtras,
    ) -> c_int;
    pub fn argus_b200_decode_step(
        ctx: *mut ArgusB200Ctx, stream: *mut c_void, q: *const f32, k_new: *const f32, v_new: *const f32,
        k_cache: *mut c_void, v_cache: *mut c_void, out: *mut f32, num_heads_q: c_int, num_heads_kv: c_int,
        head_dim: c_int, cache_seq_len: i64, capacity: i64, kv_dtype: c_int, head_stride: i64, pos_stride: i64,
        extras: *const ArgusB200DecodeExtras,
    ) -> c_int;
    pub fn argus_b200_decode_step_batched(
        ctx: *mut ArgusB200Ctx, stream: *mut c_void, q: *const f32, k_new: *const f32, v_new: *const f32,
        seqs: *const ArgusB200Seq, capacity: *const i64, n_seqs: c_int, out: *mut f32, num_heads_q: c_int,
        num_heads_kv: c_int, head_dim: c_int, kv_dtype: c_int, extras: *const ArgusB200DecodeExtras,
    ) -> c_int;
    pub fn argus_b200_kivi_attention_batched(
        ctx: *mut ArgusB200Ctx, stream: *mut c_void, q: *const f32, seqs: *const ArgusB200KiviSeq, n_seqs: c_int,
        out: *mut f32, num_heads_q: c_int, num_heads_kv: c_int, head_dim: c_int, res_cap: c_int, bits: c_int,
        res_dtype: c_int, scale: f32, extras: *const ArgusB200DecodeExtras,
    ) -> c_int;
    pub fn argus_b200_kivi_attention_paged(
        ctx: *mut ArgusB200Ctx, stream: *mut c_void, q: *const f32, qk_pool: *const c_void, qv_pool: *const c_void,
        seqs: *const ArgusB200KiviPagedSeq, n_seqs: c_int, out: *mut f32, num_heads_q: c_int, num_heads_kv: c_int,
        head_dim: c_int, res_cap: c_int, bits: c_int, res_dtype: c_int, scale: f32,
        extras: *const ArgusB200DecodeExtras,
    ) -> c_int;
    pub fn argus_b200_exchange_wait_merge(
        ctx: *mut ArgusB200Ctx, stream: *mut c_void, own_part: *const f32, exchange: *const ArgusB200Exchange, step: c_int,
        num_heads_q: c_int, num_heads_kv: c_int, head_dim: c_int, out: *mut f32,
    ) -> c_int;
    pub fn argus_b200_exchange_lines_per_head(num_heads_q: c_int, num_heads_kv: c_int, head_dim: c_int) -> c_int;
    pub fn argus_b200_attention_gen_sharded(
        ctx: *mut ArgusB200Ctx, stream: *mut c_void, q: *const f32, k_shard: *const c_void, v_shard: *const c_void,
        out: *mut f32, num_heads_q: c_int, num_heads_kv: c_int, head_dim: c_int, shard_len: i64, kv_dtype: c_int,
        head_stride: i64, pos_stride: i64, exchange: *const ArgusB200Exchange,
    ) -> c_int;
    pub fn argus_b200_static_scratch_bytes() -> usize;
    pub fn argus_b200_static_last_error() -> *const c_char;
    pub fn argus_b200_last_error(ctx: *const ArgusB200Ctx) -> *const c_char;
    pub fn argus_b200_attention_gen(
        ctx: *mut ArgusB200Ctx, stream: *mut c_void, q: *const f32, k_cache: *const c_void, v_cache: *const c_void,
        out: *mut f32, num_heads_q: c_int, num_heads_kv: c_int, head_dim: c_int, cache_seq_len: i64, kv_dtype: c_int,
        head_stride: i64, pos_stride: i64, extras: *const ArgusB200DecodeExtras,
    ) -> c_int;
    pub fn argus_b200_flash_attention_prefill(
        ctx: *mut ArgusB200Ctx, stream: *mut c_void, q: *const c_void, k_cache: *const c_void, v_cache: *const c_void,
        out: *mut c_void, n_heads_q: c_int, n_heads_kv: c_int, seq_len: c_int, cache_seq_len: c_int, head_dim: c_int,
        kv_capacity: i64, batch_size: c_int, is_head_major: c_int, dtype_mode: c_int,
    ) -> c_int;
    pub fn argus_b200_prefill_attention_scores(
        ctx: *mut ArgusB200Ctx, stream: *mut c_void, q: *const f32, k_cache: *const c_void, v_cache: *const c_void,
        kv_dtype: c_int, num_heads_q: c_int, num_heads_kv: c_int, head_dim: c_int, seq_len: c_int, cache_seq_len: c_int,
        head_stride: i64, pos_stride: i64, q_start_pos: c_int, q_window: c_int, window: c_int, sum_out: *mut f32,
        per_row: *mut f32, per_row_per_head: c_int,
    ) -> c_int;
    pub fn argus_b200_attention_gen_paged(
        ctx: *mut ArgusB200Ctx, stream: *mut c_void, q: *const f32, k_pool: *const c_void, v_pool: *const c_void,
        seqs: *const ArgusB200PagedSeq, n_seqs: c_int, out: *mut f32, num_heads_q: c_int, num_heads_kv: c_int,
        head_dim: c_int, page_tokens: c_int, page_stride: i64, head_stride: i64, pos_stride: i64,
        extras: *const ArgusB200DecodeExtras,
    ) -> c_int;
    pub fn argus_b200_kv_scatter(
        ctx: *mut ArgusB200Ctx, stream: *mut c_void, k_src: *const f32, v_src: *const f32, k_dst: *mut c_void,
        v_dst: *mut c_void, dst_dtype: c_int, num_heads_kv: c_int, head_dim: c_int, capacity: i64, head_stride: i64,
        pos_stride: i64, write_pos: i64, seq_len: i64,
    ) -> c_int;
    pub fn argus_b200_kv_scatter_batched(
        ctx: *mut ArgusB200Ctx, stream: *mut c_void, k_src: *const f32, v_src: *const f32, seqs: *const ArgusB200Seq,
        capacity: *const i64, n_seqs: c_int, dst_dtype: c_int, num_heads_kv: c_int, head_dim: c_int,
    ) -> c_int;
    pub fn argus_b200_d2o_nearest(
        ctx: *mut ArgusB200Ctx, stream: *mut c_void, k_cache: *const c_void, kv_dtype: c_int, num_heads_kv: c_int,
        head_dim: c_int, head_stride: i64, pos_stride: i64, evict_pos: *const i32, n_evict: c_int,
        retain_pos: *const i32, n_retain: c_int, nearest_out: *mut i32, sim_out: *mut f32,
    ) -> c_int;
    pub fn argus_b200_kv_compact(
        ctx: *mut ArgusB200Ctx, stream: *mut c_void, k: *mut c_void, v: *mut c_void, kv_dtype: c_int,
        num_heads_kv: c_int, head_dim: c_int, capacity: i64, head_stride: i64, pos_stride: i64, keep_dev: *const i32,
        n_keep: i64, write_start: i64, head: c_int,
    ) -> c_int;
    pub fn argus_b200_kv_snapshot_prefix(
        ctx: *mut ArgusB200Ctx, stream: *mut c_void, k: *const c_void, v: *const c_void, kv_dtype: c_int,
        num_heads_kv: c_int, head_dim: c_int, capacity: i64, head_stride: i64, pos_stride: i64, token_count: i64,
        dst: *mut c_void, dst_bytes: usize,
    ) -> c_int;
    pub fn argus_b200_kv_restore_prefix(
        ctx: *mut ArgusB200Ctx, stream: *mut c_void, k: *mut c_void, v: *mut c_void, kv_dtype: c_int,
        num_heads_kv: c_int, head_dim: c_int, capacity: i64, head_stride: i64, pos_stride: i64, token_count: i64,
        src: *const c_void, src_bytes: usize,
    ) -> c_int;
    pub fn argus_b200_kv_make_resident(ctx: *mut ArgusB200Ctx, stream: *mut c_void, ptr: *const c_void, bytes: usize) -> c_int;
    pub fn argus_b200_kv_alloc(ctx: *mut ArgusB200Ctx, bytes: usize, managed: c_int, out: *mut *mut c_void) -> c_int;
    pub fn argus_b200_kv_free(ctx: *mut ArgusB200Ctx, ptr: *mut c_void) -> c_int;
    pub fn argus_b200_kv_weighted_merge(
        ctx: *mut ArgusB200Ctx, stream: *mut c_void, k: *mut c_void, v: *mut c_void, kv_dtype: c_int,
        num_heads_kv: c_int, head_dim: c_int, head_stride: i64, pos_stride: i64, into_pos: *const i32,
        into_weight: *const f32, from_start: *const i32, from_pos: *const i32, from_weight: *const f32,
        n_merges: c_int, axis: c_int,
    ) -> c_int;
    pub fn argus_b200_kivi_has_quant_attn_kernel(ctx: *const ArgusB200Ctx, bits: c_int) -> c_int;
    pub fn argus_b200_kivi_attention_gen_quant(ctx: *mut ArgusB200Ctx, args: *const CudaQuantAttnArgs) -> c_int;
    pub fn argus_b200_kivi_gather_update_quant(ctx: *mut ArgusB200Ctx, args: *const CudaQuantAttnGatherArgs) -> c_int;
    pub fn argus_b200_kivi_dequant_flush(ctx: *mut ArgusB200Ctx, args: *const CudaQuantDequantFlushArgs) -> c_int;
    pub fn argus_b200_kivi_scatter_residual(ctx: *mut ArgusB200Ctx, args: *const CudaQuantScatterResidualArgs) -> c_int;
    pub fn argus_b200_kivi_flush_pack(
        ctx: *mut ArgusB200Ctx, stream: *mut c_void, res_k: *const f32, res_v: *const f32, qk: *mut c_void,
        qv: *mut c_void, kv_heads: c_int, head_dim: c_int, res_cap: c_int, n_groups: c_int, bits: c_int,
        k_block_start: i64, v_block_start: i64,
    ) -> c_int;
    pub fn argus_b200_score_reduce(ctx: *mut ArgusB200Ctx, args: *const CudaScoreReduceArgs) -> c_int;
    pub fn argus_b200_score_reduce_per_layer(ctx: *mut ArgusB200Ctx, args: *const CudaScoreReduceArgs) -> c_int;
    pub fn argus_b200_lse_merge(
        ctx: *mut ArgusB200Ctx, stream: *mut c_void, parts: *const f32, n_parts: c_int, part_stride: i64,
        num_heads_q: c_int, head_dim: c_int, out: *mut f32, lse_out: *mut f32,
    ) -> c_int;
    pub fn argus_b200_attention_gen_static(
        stream: *mut c_void, q: *const f32, k_cache: *const c_void, v_cache: *const c_void, out: *mut f32,
        lse: *mut f32, num_heads_q: c_int, num_heads_kv: c_int, head_dim: c_int, cache_seq_len: i64, kv_dtype: c_int,
        head_stride: i64, pos_stride: i64,
    ) -> c_int;
}

/// Owner of one library context. The engine touches it from its single inference thread only
/// (the same contract as `KiviCudaBackend`, crates/techniques/kivi/src/gpu_kivi_cuda.rs:50-53).
pub struct B200Context(*mut ArgusB200Ctx);
unsafe impl Send for B200Context {}
unsafe impl Sync for B200Context {}

impl B200Context {
    /// `cu_context` is the raw `CUcontext` the engine lends to a plugin factory (`CudaQuantAttnMakeArgs.cu_context`):
    /// the library pushes it for its allocations and pops it again; it is borrowed and never destroyed, the same
    /// contract as `CudaContext::from_raw_context` in crates/techniques/kivi/src/gpu_kivi_cuda.rs:387-399.
    pub fn new(cu_context: *mut c_void, device: i32) -> Result<Self, String> {
        if cu_context.is_null() {
            return Err("null cu_context".to_string());
        }
        let mut p = std::ptr::null_mut();
        // SAFETY: plain FFI call; the context handle stays owned by the engine.
        let rc = unsafe { argus_b200_create_in_context(cu_context, device, 0, &mut p) };
        if rc != 0 || p.is_null() {
            return Err(format!("argus_b200_create_in_context failed: {rc}"));
        }
        Ok(Self(p))
    }
    pub fn raw(&self) -> *mut ArgusB200Ctx {
        self.0
    }
    pub fn last_error(&self) -> String {
        // SAFETY: the library returns a NUL-terminated string owned by the context.
        unsafe { CStr::from_ptr(argus_b200_last_error(self.0)).to_string_lossy().into_owned() }
    }
}

impl Drop for B200Context {
    fn drop(&mut self) {
        // SAFETY: created by argus_b200_create, destroyed once.
        unsafe { argus_b200_destroy(self.0) }
    }
}

/// `--backend-cap kivi_abi` on B200: the four entry points forward the engine's own argument structs.
pub struct B200QuantAttn(B200Context);

impl CudaQuantAttnBackend for B200QuantAttn {
    fn has_quant_attn_kernel(&self, bits: u8) -> bool {
        unsafe { argus_b200_kivi_has_quant_attn_kernel(self.0.raw(), bits as c_int) != 0 }
    }
    fn is_nosub_device(&self) -> bool {
        true
    }
    fn attention_gen_quant(&self, args: &CudaQuantAttnArgs) -> i32 {
        unsafe { argus_b200_kivi_attention_gen_quant(self.0.raw(), args) }
    }
    fn gather_update_quant(&self, args: &CudaQuantAttnGatherArgs) -> i32 {
        unsafe { argus_b200_kivi_gather_update_quant(self.0.raw(), args) }
    }
    fn dequant_flush(&self, args: &CudaQuantDequantFlushArgs) -> i32 {
        unsafe { argus_b200_kivi_dequant_flush(self.0.raw(), args) }
    }
    fn scatter_residual(&self, args: &CudaQuantScatterResidualArgs) -> i32 {
        unsafe { argus_b200_kivi_scatter_residual(self.0.raw(), args) }
    }
}

fn make_quant_attn(args: &CudaQuantAttnMakeArgs) -> Result<Box<dyn CudaQuantAttnBackend>, String> {
    if args.cc_major != 10 {
        return Err(format!("argus-b200 needs an sm_100 device, got sm_{}{}", args.cc_major, args.cc_minor));
    }
    Ok(Box::new(B200QuantAttn(B200Context::new(args.cu_context, args.cu_device)?)))
}

/// Registered beside (not instead of) the JIT plugin: selected with `--backend-cap kivi_b200`.
#[distributed_slice(CUDA_QUANT_ATTN_REGS)]
static B200_QUANT_ATTN: CudaQuantAttnReg = CudaQuantAttnReg { name: "kivi_b200", make: make_quant_attn };

pub struct B200ScoreReduce(B200Context);

impl CudaScoreReduceBackend for B200ScoreReduce {
    fn name(&self) -> &str {
        "attn_score_b200"
    }
    fn reduce(&self, args: &CudaScoreReduceArgs) -> i32 {
        unsafe { argus_b200_score_reduce(self.0.raw(), args) }
    }
    fn reduce_per_layer(&self, args: &CudaScoreReduceArgs) -> i32 {
        unsafe { argus_b200_score_reduce_per_layer(self.0.raw(), args) }
    }
}

fn make_score_reduce(args: &CudaScoreReduceMakeArgs) -> Result<Box<dyn CudaScoreReduceBackend>, String> {
    Ok(Box::new(B200ScoreReduce(B200Context::new(args.cu_context, args.cu_device)?)))
}

#[distributed_slice(CUDA_SCORE_REDUCERS)]
static B200_SCORE_REDUCE: CudaScoreReduceReg = CudaScoreReduceReg { name: "attn_score_b200", make: make_score_reduce };

// Layout guards: the C header asserts the same numbers.
const _: () = assert!(std::mem::size_of::<CudaQuantAttnArgs>() == 128);
const _: () = assert!(std::mem::size_of::<CudaQuantAttnGatherArgs>() == 64);
const _: () = assert!(std::mem::size_of::<CudaQuantDequantFlushArgs>() == 72);
const _: () = assert!(std::mem::size_of::<CudaQuantScatterResidualArgs>() == 64);
const _: () = assert!(std::mem::size_of::<CudaScoreReduceArgs>() == 96);
const _: () = assert!(std::mem::size_of::<ArgusB200DecodeExtras>() == 48);
const _: () = assert!(std::mem::size_of::<ArgusB200Seq>() == 40);
const _: () = assert!(std::mem::size_of::<ArgusB200KiviSeq>() == 48);
const _: () = assert!(std::mem::size_of::<ArgusB200Exchange>() == 48);
// Field offsets of the reference's PODs, as the C header's static_asserts state them.
const _: () = assert!(std::mem::offset_of!(CudaQuantAttnArgs, scores_out) == 56);
const _: () = assert!(std::mem::offset_of!(CudaQuantAttnArgs, scores_len) == 64);
const _: () = assert!(std::mem::offset_of!(CudaQuantAttnArgs, num_heads_q) == 72);
const _: () = assert!(std::mem::offset_of!(CudaQuantAttnArgs, scale) == 120);
const _: () = assert!(std::mem::offset_of!(CudaQuantAttnArgs, bits) == 124);
const _: () = assert!(std::mem::offset_of!(CudaQuantAttnGatherArgs, kv_heads) == 24);
const _: () = assert!(std::mem::offset_of!(CudaQuantDequantFlushArgs, kv_heads) == 24);
const _: () = assert!(std::mem::offset_of!(CudaQuantDequantFlushArgs, bits) == 64);
const _: () = assert!(std::mem::offset_of!(CudaQuantDequantFlushArgs, is_key) == 65);
const _: () = assert!(std::mem::offset_of!(CudaQuantScatterResidualArgs, kv_heads) == 24);
const _: () = assert!(std::mem::offset_of!(CudaScoreReduceArgs, decay_factor) == 32);
const _: () = assert!(std::mem::offset_of!(CudaScoreReduceArgs, n_layers) == 40);
const _: () = assert!(std::mem::offset_of!(CudaScoreReduceArgs, layer_flat_importance) == 88);
const _: () = assert!(std::mem::offset_of!(ArgusB200Exchange, n_ranks) == 32);
