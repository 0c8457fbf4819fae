//! Raw FFI declarations of `libcombskv.so`, one per declaration of `include/combs_kv.h`, in the
//! header's order.  NOT COMPILED in this repository (no Rust toolchain is available where it was
//! written); `tests/test_rust_bindings.py` checks that every symbol the header declares has a
//! `pub fn` here with the same number of parameters.
//!
//! Conventions are the header's: every call returns `i32` (0 = ok, negative = error) unless it is a
//! plain counter, `cbkv_last_error()` is thread-local and borrowed, handles are `Send` but not
//! `Sync`, streams are `cudaStream_t` passed as `*mut c_void`.
#![allow(non_camel_case_types)]

use core::ffi::{c_char, c_void};

#[repr(C)]
pub struct cbkv_arena {
    _p: [u8; 0],
}
#[repr(C)]
pub struct cbkv_seq {
    _p: [u8; 0],
}
#[repr(C)]
pub struct cbkv_rope {
    _p: [u8; 0],
}
#[repr(C)]
pub struct cbkv_sessions {
    _p: [u8; 0],
}

pub const CBKV_OK: i32 = 0;
pub const CBKV_ERR_POS: i32 = -1;
pub const CBKV_ERR_CAPACITY: i32 = -2;
pub const CBKV_ERR_EXHAUSTED: i32 = -3;
pub const CBKV_ERR_ARG: i32 = -4;
pub const CBKV_ERR_CUDA: i32 = -5;
pub const CBKV_ERR_STATE: i32 = -6;
pub const CBKV_ERR_DEVICE: i32 = -7;
pub const CBKV_ERR_INTERNAL: i32 = -8;

pub const CBKV_F16: i32 = 0;
pub const CBKV_BF16: i32 = 1;

pub const CBKV_ROPE_NONE: i32 = 0;
pub const CBKV_ROPE_LINEAR: i32 = 1;
pub const CBKV_ROPE_LLAMA3: i32 = 2;
pub const CBKV_ROPE_YARN: i32 = 3;
pub const CBKV_ROPE_LONGROPE: i32 = 4;

/// `CacheConfig` (kv.rs:40-85) plus geometry and per-layer windows (kv.rs:508-527).
#[repr(C)]
#[derive(Clone, Copy)]
pub struct cbkv_config {
    pub num_layers: i32,
    pub n_q_heads: i32,
    pub n_kv_heads: i32,
    pub head_dim: i32,
    pub page_size: i32,
    pub dtype: i32,
    pub max_seq_len: i64,
    pub num_pages: i64,
    pub layer_windows: *const i64,
    pub sliding_popn_refuses: i32,
    pub device: i32,
    pub quantize_kv: i32,
}

/// `PageStats` (kv.rs:153-175), same eight counters in the same order.
#[repr(C)]
#[derive(Clone, Copy, Default)]
pub struct cbkv_page_stats_t {
    pub pages_used: i64,
    pub pages_free: i64,
    pub num_pages: i64,
    pub page_size: i64,
    pub seq_len: i64,
    pub layers_materialized: i64,
    pub layers_total: i64,
    pub layers_sliding: i64,
}

/// `RotaryEmbedding::new_scaled` + `RopeScaling` (rope.rs:31-125,160-177).
#[repr(C)]
#[derive(Clone, Copy)]
pub struct cbkv_rope_config {
    pub head_dim: i32,
    pub scaling: i32,
    pub theta: f64,
    pub max_position: i64,
    pub factor: f64,
    pub low_freq_factor: f64,
    pub high_freq_factor: f64,
    pub beta_fast: f64,
    pub beta_slow: f64,
    pub original_max_position: i64,
    pub has_attention_factor: i32,
    pub attention_factor: f64,
    pub short_factor: *const f64,
    pub n_short_factor: i32,
}

/// Per-head norm of q and k before the rotation (llama.rs:275-281, norm.rs:33-39).
#[repr(C)]
#[derive(Clone, Copy)]
pub struct cbkv_qk_norm {
    pub q_weight: *const c_void,
    pub k_weight: *const c_void,
    pub eps: f64,
    pub gemma: i32,
}

extern "C" {
    pub fn cbkv_last_error() -> *const c_char;

    // ---- construction
    pub fn cbkv_arena_create(cfg: *const cbkv_config, out: *mut *mut cbkv_arena) -> i32;
    pub fn cbkv_arena_destroy(arena: *mut cbkv_arena) -> i32;
    pub fn cbkv_set_free_list(arena: *mut cbkv_arena, ids: *const i64, n: i64) -> i32;
    pub fn cbkv_seq_create(arena: *mut cbkv_arena, out: *mut *mut cbkv_seq) -> i32;
    pub fn cbkv_seq_destroy(seq: *mut cbkv_seq) -> i32;
    pub fn cbkv_seq_fork_prefix(parent: *mut cbkv_seq, n_tokens: i64, out: *mut *mut cbkv_seq) -> i32;

    // ---- one forward pass
    pub fn cbkv_begin_step(arena: *mut cbkv_arena, seqs: *const *mut cbkv_seq, new_tokens: *const i64, pos: *const i64, n_seqs: i32, stream: *mut c_void) -> i32;
    pub fn cbkv_append(arena: *mut cbkv_arena, layer: i32, k: *const c_void, v: *const c_void, stream: *mut c_void) -> i32;
    pub fn cbkv_paged_attention(arena: *mut cbkv_arena, layer: i32, q: *const c_void, out: *mut c_void, scale: f64, window: i64, stream: *mut c_void) -> i32;
    pub fn cbkv_attention(arena: *mut cbkv_arena, layer: i32, q: *const c_void, k: *const c_void, v: *const c_void, out: *mut c_void, scale: f64, window: i64, stream: *mut c_void) -> i32;
    pub fn cbkv_attention_host(arena: *mut cbkv_arena, layer: i32, q_host: *const c_void, k_host: *const c_void, v_host: *const c_void, out_host: *mut c_void, scale: f64, window: i64, stream: *mut c_void) -> i32;
    pub fn cbkv_attention_host_async(arena: *mut cbkv_arena, layer: i32, q_host: *const c_void, k_host: *const c_void, v_host: *const c_void, out_host: *mut c_void, scale: f64, window: i64, stream: *mut c_void) -> i32;
    pub fn cbkv_host_sync(arena: *mut cbkv_arena) -> i32;
    pub fn cbkv_host_alloc(bytes: usize, out: *mut *mut c_void) -> i32;
    pub fn cbkv_host_free(p: *mut c_void) -> i32;

    // ---- rotary embedding and QK norm fused into the append
    pub fn cbkv_rope_tables_host(cfg: *const cbkv_rope_config, cos_out: *mut f32, sin_out: *mut f32) -> i32;
    pub fn cbkv_rope_inv_freq_host(cfg: *const cbkv_rope_config, inv_freq_out: *mut f64, mscale_out: *mut f64) -> i32;
    pub fn cbkv_rope_create(arena: *mut cbkv_arena, cfg: *const cbkv_rope_config, out: *mut *mut cbkv_rope) -> i32;
    pub fn cbkv_rope_destroy(rope: *mut cbkv_rope) -> i32;
    pub fn cbkv_rope_append(arena: *mut cbkv_arena, layer: i32, rope: *const cbkv_rope, norm: *const cbkv_qk_norm, q: *const c_void, k: *const c_void, v: *const c_void, q_out: *mut c_void, stream: *mut c_void) -> i32;
    pub fn cbkv_attention_rope(arena: *mut cbkv_arena, layer: i32, rope: *const cbkv_rope, norm: *const cbkv_qk_norm, q: *const c_void, k: *const c_void, v: *const c_void, out: *mut c_void, scale: f64, window: i64, stream: *mut c_void) -> i32;

    // ---- sessions, prefix reuse, speculative rollback, stats
    pub fn cbkv_sessions_create(arena: *mut cbkv_arena, max_sessions: i32, out: *mut *mut cbkv_sessions) -> i32;
    pub fn cbkv_sessions_destroy(set: *mut cbkv_sessions) -> i32;
    pub fn cbkv_sessions_acquire(set: *mut cbkv_sessions, key: *const c_char, prompt: *const u32, n_prompt: i64, reuse: i32, seq_out: *mut *mut cbkv_seq, lcp_out: *mut i64) -> i32;
    pub fn cbkv_sessions_release(set: *mut cbkv_sessions, key: *const c_char, seq: *mut cbkv_seq, history: *const u32, n_history: i64, reuse: i32) -> i32;
    pub fn cbkv_sessions_clear(set: *mut cbkv_sessions, removed: *mut i64) -> i32;
    pub fn cbkv_sessions_count(set: *const cbkv_sessions) -> i64;
    pub fn cbkv_sessions_evictions(set: *const cbkv_sessions) -> i64;
    pub fn cbkv_sessions_history_len(set: *const cbkv_sessions, key: *const c_char) -> i64;
    pub fn cbkv_spec_verify_rollback(seq: *mut cbkv_seq, draft: *const u32, argmax: *const u32, k: i32, accepted_out: *mut i32, correction_out: *mut u32) -> i32;
    pub fn cbkv_sessions_stats_json(set: *const cbkv_sessions, buf: *mut c_char, cap: i64) -> i64;

    // ---- decode attention that allocates nothing (no reference counterpart)
    pub fn cbkv_decode_attention_static(kv_pages: *const c_void, num_pages: i64, block_tables: *const i32, table_stride: i32, seq_lens_host: *const i32, n_seqs: i32, n_q_heads: i32, n_kv_heads: i32, head_dim: i32, dtype: i32, q: *const c_void, out: *mut c_void, scale: f64, window: i64, stream: *mut c_void) -> i32;
    pub fn cbkv_static_status(stream: *mut c_void, status: *mut i32) -> i32;

    // ---- rollback / reset / counters
    pub fn cbkv_popn(seq: *mut cbkv_seq, n: i64, popped: *mut i64) -> i32;
    pub fn cbkv_reset(seq: *mut cbkv_seq) -> i32;
    pub fn cbkv_seq_len(seq: *const cbkv_seq) -> i64;
    pub fn cbkv_pages_used(seq: *const cbkv_seq) -> i64;
    pub fn cbkv_num_free_pages(arena: *const cbkv_arena) -> i64;
    pub fn cbkv_page_stats(seq: *const cbkv_seq, out: *mut cbkv_page_stats_t) -> i32;
    pub fn cbkv_page_bytes(arena: *const cbkv_arena) -> i64;

    // ---- state export
    pub fn cbkv_export_block_table(seq: *const cbkv_seq, out: *mut i64, cap: i64) -> i64;
    pub fn cbkv_export_free_list(arena: *const cbkv_arena, out: *mut i64, cap: i64) -> i64;
    pub fn cbkv_export_page(arena: *mut cbkv_arena, layer: i32, page: i64, k_out_host: *mut c_void, v_out_host: *mut c_void, stream: *mut c_void) -> i32;
    pub fn cbkv_export_page_quant(arena: *mut cbkv_arena, layer: i32, page: i64, k_packed_host: *mut i32, k_scales_host: *mut c_void, v_packed_host: *mut i32, v_scales_host: *mut c_void, stream: *mut c_void) -> i32;
    pub fn cbkv_layer_is_quantized(arena: *const cbkv_arena, layer: i32) -> i32;
    pub fn cbkv_page_refcount(arena: *const cbkv_arena, page: i64) -> i32;

    // ---- diagnostics and tuning
    pub fn cbkv_device_status(arena: *mut cbkv_arena, stream: *mut c_void, status: *mut i32) -> i32;
    pub fn cbkv_launch_count() -> i64;
    pub fn cbkv_profile_enable(arena: *mut cbkv_arena, on: i32) -> i32;
    pub fn cbkv_profile_read(arena: *mut cbkv_arena, total_ms: *mut f64, launches: *mut i64) -> i32;
    pub fn cbkv_set_decode_tuning(arena: *mut cbkv_arena, ctas_per_sm: i32, stages: i32, consumers: i32, max_ctas: i32, overlap_launches: i32) -> i32;
    pub fn cbkv_set_host_route(arena: *mut cbkv_arena, direct: i32) -> i32;
    pub fn cbkv_set_chunk_split(arena: *mut cbkv_arena, max_parts: i32) -> i32;
    pub fn cbkv_set_chunk_kernel(arena: *mut cbkv_arena, mode: i32) -> i32;
    pub fn cbkv_set_decode_split(arena: *mut cbkv_arena, tail_pct: i32, min_item: i32, max_levels: i32) -> i32;

    // ---- test hooks
    pub fn cbkv_debug_begin_step_host(arena: *mut cbkv_arena, seqs: *const *mut cbkv_seq, new_tokens: *const i64, pos: *const i64, n_seqs: i32) -> i32;
    pub fn cbkv_debug_decode_plan(arena: *mut cbkv_arena, window: i64, n_ctas: i32, tail_pct: i32, min_item: i32, out: *mut i32, cap: i64) -> i64;
    pub fn cbkv_debug_set_wait_limit(arena: *mut cbkv_arena, wait_us: i64, fault_tile: i32) -> i32;
    pub fn cbkv_debug_raise(kind: i32) -> i32;
}
