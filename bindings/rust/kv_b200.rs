//! `impl KVCache` over `libcombskv.so`: the file a maintainer drops into
//! `engine/core/combs-models/src/` next to `kv.rs`.  NOT COMPILED in this repository (no Rust
//! toolchain where it was written); it is the binding the C ABI was shaped for, kept as a file so
//! that it can be reviewed and built, not a tested product path.
//!
//! One `B200PagedKVCache` is one reference `PagedKVCache` (kv.rs:477-855): a single sequence over a
//! private arena.  `B` must be a backend whose tensors expose a CUDA device pointer and the stream
//! they are ordered on (`CudaBackend` below states exactly what is needed).
use core::ffi::c_void;
use std::ffi::CStr;
use std::ptr;

use burn::tensor::{backend::Backend, Tensor};
use combs_kv_sys::*;

use crate::kv::{CacheConfig, KVCache, PageStats};

/// What the binding needs from a backend: raw device pointers of contiguous f16 tensors and the
/// CUDA stream the backend enqueues on.
pub trait CudaBackend: Backend {
    fn cuda_ptr<const D: usize>(t: &Tensor<Self, D>) -> *const c_void;
    fn cuda_ptr_mut<const D: usize>(t: &mut Tensor<Self, D>) -> *mut c_void;
    fn cuda_stream(device: &Self::Device) -> *mut c_void;
    fn device_ordinal(device: &Self::Device) -> i32;
}

pub struct B200PagedKVCache {
    arena: *mut cbkv_arena,
    seq: *mut cbkv_seq,
    stream: *mut c_void,
}

// The trait is Send, not Sync (kv.rs:92): the handles may move between threads, one owner at a time.
unsafe impl Send for B200PagedKVCache {}

fn last_error() -> String {
    unsafe { CStr::from_ptr(cbkv_last_error()) }.to_string_lossy().into_owned()
}

/// The library keeps the reference's panic texts in `cbkv_last_error`, so re-panicking with them
/// reproduces the reference's failure behaviour (kv.rs:552-555,671-683).
fn check(rc: i32) {
    if rc != CBKV_OK {
        panic!("{}", last_error());
    }
}

impl B200PagedKVCache {
    /// `PagedKVCache::new_with_windows` (kv.rs:508-527).
    pub fn new_with_windows<B: CudaBackend>(
        num_layers: usize,
        n_q_heads: usize,
        n_kv_heads: usize,
        head_dim: usize,
        cfg: &CacheConfig,
        windows: &[Option<usize>],
        device: &B::Device,
    ) -> Self {
        assert_eq!(windows.len(), num_layers, "one window entry per layer"); // kv.rs:513
        let w: Vec<i64> = windows.iter().map(|w| w.map_or(0, |x| x as i64)).collect();
        let c = cbkv_config {
            num_layers: num_layers as i32,
            n_q_heads: n_q_heads as i32,
            n_kv_heads: n_kv_heads as i32,
            head_dim: head_dim as i32,
            page_size: cfg.page_size as i32,
            dtype: CBKV_F16,
            max_seq_len: cfg.max_seq_len as i64,
            num_pages: 0,
            layer_windows: w.as_ptr(),
            sliding_popn_refuses: 1,
            device: B::device_ordinal(device),
            quantize_kv: cfg.quantize_kv as i32,
        };
        let mut arena = ptr::null_mut();
        check(unsafe { cbkv_arena_create(&c, &mut arena) });
        let mut seq = ptr::null_mut();
        check(unsafe { cbkv_seq_create(arena, &mut seq) });
        Self { arena, seq, stream: B::cuda_stream(device) }
    }

    /// Inherent `num_free_pages` (kv.rs:529-532).
    pub fn num_free_pages(&self) -> usize {
        unsafe { cbkv_num_free_pages(self.arena) as usize }
    }

    /// The kernels report problems in a status word instead of trapping; poll it once per step.
    pub fn device_status(&mut self) -> i32 {
        let mut st = 0i32;
        let rc = unsafe { cbkv_device_status(self.arena, self.stream, &mut st) };
        if rc != CBKV_OK && rc != CBKV_ERR_DEVICE {
            check(rc);
        }
        st
    }
}

impl<B: CudaBackend> KVCache<B> for B200PagedKVCache {
    fn attention_opts(
        &mut self,
        layer: usize,
        q: Tensor<B, 4>,
        k: Tensor<B, 4>,
        v: Tensor<B, 4>,
        pos: usize,
        scale: f64,
        window: Option<usize>,
    ) -> Tensor<B, 4> {
        let seq = k.dims()[2] as i64;
        if layer == 0 {
            // layer 0 advances the sequence and checks pos == seq_len (kv.rs:665-683)
            let p = pos as i64;
            check(unsafe { cbkv_begin_step(self.arena, &self.seq, &seq, &p, 1, self.stream) });
        }
        let mut out = Tensor::<B, 4>::empty(q.dims(), &q.device());
        check(unsafe {
            cbkv_attention(
                self.arena,
                layer as i32,
                B::cuda_ptr(&q),
                B::cuda_ptr(&k),
                B::cuda_ptr(&v),
                B::cuda_ptr_mut(&mut out),
                scale,
                window.unwrap_or(0) as i64,
                self.stream,
            )
        });
        out
    }

    fn seq_len(&self) -> usize {
        unsafe { cbkv_seq_len(self.seq) as usize }
    }

    fn popn(&mut self, n: usize) -> usize {
        let mut popped = 0i64;
        check(unsafe { cbkv_popn(self.seq, n as i64, &mut popped) });
        popped as usize
    }

    fn reset(&mut self) {
        check(unsafe { cbkv_reset(self.seq) })
    }

    fn pages_used(&self) -> Option<usize> {
        Some(unsafe { cbkv_pages_used(self.seq) as usize })
    }

    fn page_stats(&self) -> Option<PageStats> {
        let mut s = cbkv_page_stats_t::default();
        check(unsafe { cbkv_page_stats(self.seq, &mut s) });
        Some(PageStats {
            pages_used: s.pages_used as usize,
            pages_free: s.pages_free as usize,
            num_pages: s.num_pages as usize,
            page_size: s.page_size as usize,
            seq_len: s.seq_len as usize,
            layers_materialized: s.layers_materialized as usize,
            layers_total: s.layers_total as usize,
            layers_sliding: s.layers_sliding as usize,
        })
    }
}

impl Drop for B200PagedKVCache {
    fn drop(&mut self) {
        unsafe {
            cbkv_seq_destroy(self.seq);
            cbkv_arena_destroy(self.arena);
        }
    }
}
