//! Declarations of the C ABI of libqeng (include/qeng.h) for a Rust host.
//!
//! cyb reaches its model runtime through `soma_kernel::Soma` (shell/src/worlds/soma_bridge.rs:65,
//! 144-146, 242; shell/src/worlds/models/mod.rs:379-386), which drives glia `run`; a `run` backend
//! for B200 binds these symbols.  One `extern "C"` item per function of the header, same names,
//! same argument order.  NOT COMPILED HERE: the image that built the library carries no Rust
//! toolchain, so this file is checked only for naming every symbol the header declares
//! (tests/test_abi.py); link with `-lqeng`.
#![allow(non_camel_case_types)]

use std::os::raw::{c_char, c_void};

#[repr(C)]
pub struct qeng_ctx {
    _private: [u8; 0],
}
#[repr(C)]
pub struct qeng_weight {
    _private: [u8; 0],
}
#[repr(C)]
pub struct qeng_kv_pool {
    _private: [u8; 0],
}
#[repr(C)]
pub struct qeng_decoder {
    _private: [u8; 0],
}

pub const QENG_OK: i32 = 0;
pub const QENG_ERR_ARG: i32 = -1;
pub const QENG_ERR_SHAPE: i32 = -2;
pub const QENG_ERR_ALIGN: i32 = -3;
pub const QENG_ERR_CUDA: i32 = -4;
pub const QENG_ERR_NCCL: i32 = -5;
pub const QENG_ERR_TIMEOUT: i32 = -6;
pub const QENG_ERR_DEVICE_STATUS: i32 = -7;
pub const QENG_ERR_STATE: i32 = -8;

pub const QENG_F32: i32 = 0;
pub const QENG_F16: i32 = 1;
pub const QENG_BF16: i32 = 2;

pub const QENG_GEMM_ACCUMULATE: i32 = 1;
pub const QENG_GEMM_FAST_F16: i32 = 2;

pub const QENG_W_Q: i32 = 0;
pub const QENG_W_K: i32 = 1;
pub const QENG_W_V: i32 = 2;
pub const QENG_W_O: i32 = 3;
pub const QENG_W_GATE: i32 = 4;
pub const QENG_W_UP: i32 = 5;
pub const QENG_W_DOWN: i32 = 6;

/// Tuning switches fixed at context creation; zero-initialise, set `struct_size`.
#[repr(C)]
#[derive(Clone, Copy, Default)]
pub struct qeng_options {
    pub struct_size: i32,
    pub no_pdl: i32,
    pub no_l2_prefetch: i32,
    pub no_p2p_allreduce: i32,
    pub no_attn_cluster: i32,
    pub attn_ctas_per_sm: i32,
    pub stream_groups: i32,
    pub step_kernel: i32,
    pub stream_stage_chunks: i32,
}

#[repr(C)]
#[derive(Clone, Copy, Default)]
pub struct qeng_model_cfg {
    pub layers: i32,
    pub d_model: i32,
    pub ffn: i32,
    pub heads: i32,
    pub kv_heads: i32,
    pub head_dim: i32,
    pub vocab: i32,
    pub rms_eps: f32,
    pub rope_base: f32,
    pub max_batch: i32,
    pub max_seq: i32,
    pub tp_rank: i32,
    pub tp_world: i32,
    pub attn_softcap: f32,
    pub sliding_window: i32,
    pub final_softcap: f32,
}

#[link(name = "qeng")]
extern "C" {
    pub fn qeng_version() -> i32;
    pub fn qeng_create(device: i32, out: *mut *mut qeng_ctx) -> i32;
    pub fn qeng_create_opts(device: i32, opts: *const qeng_options, out: *mut *mut qeng_ctx) -> i32;
    pub fn qeng_destroy(ctx: *mut qeng_ctx) -> i32;
    pub fn qeng_last_error(ctx: *const qeng_ctx) -> *const c_char;
    pub fn qeng_device_status(ctx: *mut qeng_ctx) -> i32;
    pub fn qeng_sm_count(ctx: *const qeng_ctx) -> i32;
    pub fn qeng_tp_unique_id(out128: *mut u8) -> i32;
    pub fn qeng_tp_init(ctx: *mut qeng_ctx, rank: i32, world: i32, id128: *const u8) -> i32;
    pub fn qeng_tp_p2p_handle(ctx: *mut qeng_ctx, out64: *mut u8) -> i32;
    pub fn qeng_tp_p2p_open(ctx: *mut qeng_ctx, handles: *const u8) -> i32;
    pub fn qeng_tp_p2p_reset(ctx: *mut qeng_ctx) -> i32;
    pub fn qeng_tp_all_reduce_add_f32(ctx: *mut qeng_ctx, dst: *mut f32, part: *mut f32, n: i64, stream: *mut c_void) -> i32;
    pub fn qeng_tp_all_reduce_f32(ctx: *mut qeng_ctx, buf: *mut f32, n: i64, stream: *mut c_void) -> i32;
    pub fn qeng_weight_pack_q4(ctx: *mut qeng_ctx, q: *const u8, s: *const u16, N: i64, K: i64, out: *mut *mut qeng_weight) -> i32;
    pub fn qeng_weight_unpack_q4(ctx: *mut qeng_ctx, w: *const qeng_weight, q: *mut u8, s: *mut u16) -> i32;
    pub fn qeng_weight_dequant_f32(ctx: *mut qeng_ctx, w: *const qeng_weight, out: *mut f32, stream: *mut c_void) -> i32;
    pub fn qeng_weight_quantize_q4(ctx: *mut qeng_ctx, w_dev: *const c_void, x_dtype: i32, N: i64, K: i64, ld: i64, out: *mut *mut qeng_weight, stream: *mut c_void) -> i32;
    pub fn qeng_weight_pack_q4k(ctx: *mut qeng_ctx, blocks: *const u8, N: i64, K: i64, out: *mut *mut qeng_weight) -> i32;
    pub fn qeng_weight_unpack_k4(ctx: *mut qeng_ctx, w: *const qeng_weight, q: *mut u8, scale_min: *mut f32) -> i32;
    pub fn qeng_weight_pack_q8(ctx: *mut qeng_ctx, q: *const i8, s: *const u16, N: i64, K: i64, out: *mut *mut qeng_weight) -> i32;
    pub fn qeng_weight_unpack_q8(ctx: *mut qeng_ctx, w: *const qeng_weight, q: *mut i8, s: *mut u16) -> i32;
    pub fn qeng_weight_quantize_q8(ctx: *mut qeng_ctx, w_dev: *const c_void, x_dtype: i32, N: i64, K: i64, ld: i64, out: *mut *mut qeng_weight, stream: *mut c_void) -> i32;
    pub fn qeng_weight_free(ctx: *mut qeng_ctx, w: *mut qeng_weight) -> i32;
    pub fn qeng_weight_rows(w: *const qeng_weight) -> i64;
    pub fn qeng_weight_cols(w: *const qeng_weight) -> i64;
    pub fn qeng_weight_device_bytes(w: *const qeng_weight) -> i64;
    pub fn qeng_weight_format(w: *const qeng_weight) -> i32;
    pub fn qeng_weight_set_next(ctx: *mut qeng_ctx, w: *mut qeng_weight, next: *const qeng_weight) -> i32;
    pub fn qeng_gemm_q4(ctx: *mut qeng_ctx, w: *const qeng_weight, x: *const c_void, x_dtype: i32, M: i64, ldx: i64, y: *mut f32, ldy: i64, flags: i32, stream: *mut c_void) -> i32;
    pub fn qeng_gemv_q4(ctx: *mut qeng_ctx, w: *const qeng_weight, x: *const f32, y: *mut f32, stream: *mut c_void) -> i32;
    pub fn qeng_rmsnorm(ctx: *mut qeng_ctx, x: *const f32, gamma: *const f32, M: i64, D: i64, eps: f32, y: *mut f32, stream: *mut c_void) -> i32;
    pub fn qeng_rope(ctx: *mut qeng_ctx, x: *mut f32, pos: *const i32, M: i64, H: i64, hd: i64, base: f32, stream: *mut c_void) -> i32;
    pub fn qeng_swiglu(ctx: *mut qeng_ctx, gate: *const f32, up: *const f32, n: i64, y: *mut f32, stream: *mut c_void) -> i32;
    pub fn qeng_add(ctx: *mut qeng_ctx, a: *const f32, b: *const f32, n: i64, y: *mut f32, stream: *mut c_void) -> i32;
    pub fn qeng_embed(ctx: *mut qeng_ctx, table_bf16: *const u16, tokens: *const i32, M: i64, D: i64, V: i64, x: *mut f32, stream: *mut c_void) -> i32;
    pub fn qeng_lm_head(ctx: *mut qeng_ctx, table_bf16: *const u16, x: *const f32, M: i64, D: i64, V: i64, logits: *mut f32, stream: *mut c_void) -> i32;
    pub fn qeng_argmax(ctx: *mut qeng_ctx, logits: *const f32, M: i64, V: i64, idx: *mut i32, stream: *mut c_void) -> i32;
    pub fn qeng_kv_pool_create(ctx: *mut qeng_ctx, pages: i64, kv_heads: i64, hd: i64, out: *mut *mut qeng_kv_pool) -> i32;
    pub fn qeng_kv_pool_free(ctx: *mut qeng_ctx, pool: *mut qeng_kv_pool) -> i32;
    pub fn qeng_kv_pool_data(pool: *const qeng_kv_pool) -> *mut c_void;
    pub fn qeng_kv_pool_pages(pool: *const qeng_kv_pool) -> i64;
    pub fn qeng_kv_append(ctx: *mut qeng_ctx, pool: *mut qeng_kv_pool, k: *const f32, v: *const f32, page_table: *const i32, max_pages: i64, pos: *const i32, B: i64, stream: *mut c_void) -> i32;
    pub fn qeng_attn_decode(ctx: *mut qeng_ctx, pool: *const qeng_kv_pool, q_f16: *const u16, page_table: *const i32, max_pages: i64, lens: *const i32, B: i64, Hq: i64, scale: f32, out: *mut f32, stream: *mut c_void) -> i32;
    pub fn qeng_attn_decode_ex(ctx: *mut qeng_ctx, pool: *const qeng_kv_pool, q_f16: *const u16, page_table: *const i32, max_pages: i64, lens: *const i32, B: i64, Hq: i64, scale: f32, softcap: f32, window: i32, out: *mut f32, stream: *mut c_void) -> i32;
    pub fn qeng_attn_decode_noalloc(ctx: *mut qeng_ctx, pool: *const qeng_kv_pool, q_f16: *const u16, page_table: *const i32, max_pages: i64, lens: *const i32, B: i64, Hq: i64, scale: f32, out: *mut f32, stream: *mut c_void) -> i32;
    pub fn qeng_decoder_create(ctx: *mut qeng_ctx, cfg: *const qeng_model_cfg, out: *mut *mut qeng_decoder) -> i32;
    pub fn qeng_decoder_free(ctx: *mut qeng_ctx, dec: *mut qeng_decoder) -> i32;
    pub fn qeng_decoder_load_matrix(ctx: *mut qeng_ctx, dec: *mut qeng_decoder, layer: i32, which: i32, q: *const u8, s: *const u16, N: i64, K: i64) -> i32;
    pub fn qeng_decoder_load_matrix_q8(ctx: *mut qeng_ctx, dec: *mut qeng_decoder, layer: i32, which: i32, q: *const i8, s: *const u16, N: i64, K: i64) -> i32;
    pub fn qeng_decoder_load_matrix_q4k(ctx: *mut qeng_ctx, dec: *mut qeng_decoder, layer: i32, which: i32, blocks: *const u8, N: i64, K: i64) -> i32;
    pub fn qeng_decoder_load_norm(ctx: *mut qeng_ctx, dec: *mut qeng_decoder, layer: i32, which: i32, gamma: *const f32) -> i32;
    pub fn qeng_decoder_load_head(ctx: *mut qeng_ctx, dec: *mut qeng_decoder, emb: *const u16, lm_head: *const u16, final_gamma: *const f32) -> i32;
    pub fn qeng_decoder_config(ctx: *mut qeng_ctx, dec: *const qeng_decoder, out: *mut qeng_model_cfg) -> i32;
    pub fn qeng_model_file_config(ctx: *mut qeng_ctx, path: *const c_char, out: *mut qeng_model_cfg, n_tensors: *mut i64) -> i32;
    pub fn qeng_decoder_load_file(ctx: *mut qeng_ctx, dec: *mut qeng_decoder, path: *const c_char) -> i32;
    pub fn qeng_decoder_reset(ctx: *mut qeng_ctx, dec: *mut qeng_decoder, batch: i32) -> i32;
    pub fn qeng_decoder_prefill(ctx: *mut qeng_ctx, dec: *mut qeng_decoder, tokens: *const i32, batch: i32, T: i32) -> i32;
    pub fn qeng_decoder_decode(ctx: *mut qeng_ctx, dec: *mut qeng_decoder, steps: i32, out_tokens: *mut i32) -> i32;
    pub fn qeng_decoder_logits(ctx: *mut qeng_ctx, dec: *mut qeng_decoder, out: *mut f32) -> i32;
    pub fn qeng_decoder_layer(ctx: *mut qeng_ctx, dec: *mut qeng_decoder, layer: i32, x_in: *const f32, pos: *const i32, batch: i32, x_out: *mut f32, stream: *mut c_void) -> i32;
    pub fn qeng_decoder_set_stream(ctx: *mut qeng_ctx, dec: *mut qeng_decoder, stream: *mut c_void) -> i32;
    pub fn qeng_decoder_weight(ctx: *mut qeng_ctx, dec: *mut qeng_decoder, layer: i32, fused_index: i32, out: *mut *const qeng_weight) -> i32;
    pub fn qeng_decoder_launches_per_step(dec: *const qeng_decoder) -> i32;
    pub fn qeng_decoder_step_profile(ctx: *mut qeng_ctx, dec: *mut qeng_decoder, out_ns: *mut u64, capacity: i32, n_written: *mut i32) -> i32;
}
