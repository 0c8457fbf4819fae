"""Host-side mirror of the reference's KV-cache operator surface.

Names, argument meaning and error behaviour follow
``engine/core/combs-models/src/kv.rs``: ``CacheConfig`` (kv.rs:40-85),
``PageStats`` (kv.rs:153-175), the ``KVCache`` trait (kv.rs:92-151) and
``PagedKVCache`` (kv.rs:477-855).  Where the reference panics, these raise
``CbkvError`` carrying the same message.  All compute goes through the C ABI of
``libcombskv.so``; torch is used for device memory and streams only.
"""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

from . import _lib
from ._lib import CbkvError, check

P = C.c_void_p


class CacheKind(enum.Enum):
    """kv.rs:31-38."""
    Contiguous = 0
    Paged = 1


@dataclass
class CacheConfig:
    """kv.rs:40-85."""
    max_seq_len: int
    page_size: int = 16
    kind: CacheKind = CacheKind.Paged
    quantize_kv: bool = False

    DEFAULT_PAGE_SIZE = 16

    @staticmethod
    def paged(max_seq_len: int) -> "CacheConfig":
        return CacheConfig(max_seq_len, CacheConfig.DEFAULT_PAGE_SIZE, CacheKind.Paged, False)

    @staticmethod
    def contiguous(max_seq_len: int) -> "CacheConfig":
        return CacheConfig(max_seq_len, CacheConfig.DEFAULT_PAGE_SIZE, CacheKind.Contiguous, False)

    def num_pages(self) -> int:
        return -(-self.max_seq_len // self.page_size)


@dataclass(frozen=True)
class PageStats:
    """kv.rs:153-175."""
    pages_used: int
    pages_free: int
    num_pages: int
    page_size: int
    seq_len: int
    layers_materialized: int
    layers_total: int
    layers_sliding: int


_DTYPES = {torch.float16: 0, torch.bfloat16: 1}


def _stream_ptr(stream: Optional[torch.cuda.Stream]) -> int:
    if stream is None:
        stream = torch.cuda.current_stream()
    return stream.cuda_stream


class PagedSeq:
    """One sequence over an arena: its block table and length (one reference PagedKVCache)."""

    def __init__(self, arena: "KVArena", handle: int):
        self.arena, self._h = arena, handle
        arena._seqs.add(self)

    def close(self) -> None:
        if self._h:
            check(self.arena._lib.cbkv_seq_destroy(self._h))
            self._h = None
            self.arena._seqs.discard(self)

    def fork_prefix(self, n_tokens: int) -> "PagedSeq":
        out = P()
        check(self.arena._lib.cbkv_seq_fork_prefix(self._h, n_tokens, C.byref(out)))
        return PagedSeq(self.arena, out.value)

    def popn(self, n: int) -> int:
        """kv.rs:807-835: tokens actually dropped; 0 = refused."""
        popped = C.c_int64(0)
        check(self.arena._lib.cbkv_popn(self._h, n, C.byref(popped)))
        return popped.value

    def reset(self) -> None:
        check(self.arena._lib.cbkv_reset(self._h))

    def seq_len(self) -> int:
        return self.arena._lib.cbkv_seq_len(self._h)

    def pages_used(self) -> int:
        return self.arena._lib.cbkv_pages_used(self._h)

    def page_stats(self) -> PageStats:
        st = _lib.cbkv_page_stats_t()
        check(self.arena._lib.cbkv_page_stats(self._h, C.byref(st)))
        return PageStats(*(getattr(st, f) for f, _ in st._fields_))

    def block_table(self) -> np.ndarray:
        n = self.pages_used()
        out = np.zeros(max(n, 1), dtype=np.int64)
        self.arena._lib.cbkv_export_block_table(self._h, out.ctypes.data_as(C.POINTER(C.c_int64)), len(out))
        return out[:n]


class KVArena:
    """Page arenas + LIFO free-list shared by the sequences created from it."""

    def __init__(self, num_layers: int, n_q_heads: int, n_kv_heads: int, head_dim: int, max_seq_len: int,
                 page_size: int = 16, num_pages: int = 0, windows: Optional[Sequence[Optional[int]]] = None,
                 dtype: torch.dtype = torch.float16, device: int = 0, sliding_popn_refuses: bool = True,
                 quantize_kv: bool = False):
        self._lib = _lib.load()
        if windows is not None and len(windows) != num_layers:
            raise CbkvError(-4, "one window entry per layer")  # kv.rs:513
        if dtype not in _DTYPES:
            raise CbkvError(-4, "dtype must be torch.float16 or torch.bfloat16")
        cfg = _lib.cbkv_config()
        cfg.num_layers, cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim = num_layers, n_q_heads, n_kv_heads, head_dim
        cfg.page_size, cfg.dtype, cfg.max_seq_len, cfg.num_pages = page_size, _DTYPES[dtype], max_seq_len, num_pages
        self._wbuf = None
        if windows is not None:
            self._wbuf = (C.c_int64 * num_layers)(*[0 if w is None else int(w) for w in windows])
            cfg.layer_windows = C.cast(self._wbuf, C.POINTER(C.c_int64))
        cfg.sliding_popn_refuses = 1 if sliding_popn_refuses else 0
        cfg.device = device
        cfg.quantize_kv = 1 if quantize_kv else 0   # CacheConfig::quantize_kv, kv.rs:464-475
        h = P()
        check(self._lib.cbkv_arena_create(C.byref(cfg), C.byref(h)))
        self._h = h.value
        self._seqs: set[PagedSeq] = set()
        self.num_layers, self.n_q_heads, self.n_kv_heads, self.head_dim = num_layers, n_q_heads, n_kv_heads, head_dim
        self.page_size, self.dtype, self.device = page_size, dtype, device
        self.max_seq_len = max_seq_len
        self.num_pages = num_pages if num_pages > 0 else -(-max_seq_len // page_size)
        self.step_tokens = 0

    def close(self) -> None:
        if self._h:
            for s in list(self._seqs):
                s._h = None  # the arena frees its sequences
            self._seqs.clear()
            self._lib.cbkv_arena_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- construction
    def set_free_list(self, ids) -> None:
        a = np.ascontiguousarray(ids, dtype=np.int64)
        check(self._lib.cbkv_set_free_list(self._h, a.ctypes.data_as(C.POINTER(C.c_int64)), len(a)))

    def new_seq(self) -> PagedSeq:
        out = P()
        check(self._lib.cbkv_seq_create(self._h, C.byref(out)))
        return PagedSeq(self, out.value)

    # ---- one forward pass
    def _step_args(self, seqs, new_tokens, pos):
        n = len(seqs)
        hs = (P * n)(*[s._h for s in seqs])
        nt = (C.c_int64 * n)(*[int(x) for x in new_tokens])
        ps = None if pos is None else (C.c_int64 * n)(*[int(x) for x in pos])
        return n, hs, nt, ps

    def begin_step(self, seqs: Sequence[PagedSeq], new_tokens: Sequence[int], pos: Optional[Sequence[int]] = None,
                   stream: Optional[torch.cuda.Stream] = None) -> None:
        n, hs, nt, ps = self._step_args(seqs, new_tokens, pos)
        check(self._lib.cbkv_begin_step(self._h, hs, nt, ps, n, _stream_ptr(stream)))
        self.step_tokens = int(sum(int(x) for x in new_tokens))

    def begin_step_host_only(self, seqs, new_tokens, pos=None) -> None:
        """Bookkeeping alone, no device (test hook)."""
        n, hs, nt, ps = self._step_args(seqs, new_tokens, pos)
        check(self._lib.cbkv_debug_begin_step_host(self._h, hs, nt, ps, n))
        self.step_tokens = int(sum(int(x) for x in new_tokens))

    def _chk(self, t: torch.Tensor, heads: int, name: str) -> None:
        if not (t.is_cuda and t.is_contiguous() and t.dtype == self.dtype):
            raise CbkvError(-4, f"{name} must be a contiguous {self.dtype} CUDA tensor")
        if t.numel() != self.step_tokens * heads * self.head_dim:
            raise CbkvError(-4, f"{name} has {t.numel()} elements, the step needs {self.step_tokens * heads * self.head_dim}")

    def attention(self, layer: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                  window: Optional[int] = None, out: Optional[torch.Tensor] = None,
                  stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
        """attention_opts for every sequence of the step: append + attention (kv.rs:655-791)."""
        self._chk(q, self.n_q_heads, "q"); self._chk(k, self.n_kv_heads, "k"); self._chk(v, self.n_kv_heads, "v")
        if out is None:
            out = torch.empty_like(q)
        check(self._lib.cbkv_attention(self._h, layer, q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                       float(scale), 0 if window is None else int(window), _stream_ptr(stream)))
        return out

    def append(self, layer: int, k: torch.Tensor, v: torch.Tensor, stream=None) -> None:
        self._chk(k, self.n_kv_heads, "k"); self._chk(v, self.n_kv_heads, "v")
        check(self._lib.cbkv_append(self._h, layer, k.data_ptr(), v.data_ptr(), _stream_ptr(stream)))

    def paged_attention(self, layer: int, q: torch.Tensor, scale: float, window: Optional[int] = None,
                        out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
        self._chk(q, self.n_q_heads, "q")
        if out is None:
            out = torch.empty_like(q)
        check(self._lib.cbkv_paged_attention(self._h, layer, q.data_ptr(), out.data_ptr(), float(scale),
                                             0 if window is None else int(window), _stream_ptr(stream)))
        return out

    def attention_host(self, layer: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor,
                       scale: float, window: Optional[int] = None, stream=None) -> torch.Tensor:
        """Same call with host tensors (pinned ones copy asynchronously); waits for `out`."""
        for t in (q, k, v, out):
            if t.is_cuda or not t.is_contiguous() or t.dtype != self.dtype:
                raise CbkvError(-4, "attention_host takes contiguous host tensors of the arena dtype")
        check(self._lib.cbkv_attention_host(self._h, layer, q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                            float(scale), 0 if window is None else int(window), _stream_ptr(stream)))
        return out

    def attention_host_async(self, layer: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor,
                             scale: float, window: Optional[int] = None, stream=None) -> None:
        """attention_host without the wait; `out` is valid after host_sync()."""
        for t in (q, k, v, out):
            if t.is_cuda or not t.is_contiguous() or t.dtype != self.dtype:
                raise CbkvError(-4, "attention_host_async takes contiguous host tensors of the arena dtype")
        check(self._lib.cbkv_attention_host_async(self._h, layer, q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                                  out.data_ptr(), float(scale), 0 if window is None else int(window),
                                                  _stream_ptr(stream)))

    def host_sync(self) -> None:
        check(self._lib.cbkv_host_sync(self._h))

    # ---- counters / export
    def num_free_pages(self) -> int:
        return self._lib.cbkv_num_free_pages(self._h)

    def page_bytes(self) -> int:
        return self._lib.cbkv_page_bytes(self._h)

    def free_list(self) -> np.ndarray:
        out = np.zeros(max(self.num_pages, 1), dtype=np.int64)
        n = self._lib.cbkv_export_free_list(self._h, out.ctypes.data_as(C.POINTER(C.c_int64)), len(out))
        return out[:n]

    def refcount(self, page: int) -> int:
        return self._lib.cbkv_page_refcount(self._h, page)

    def layer_is_quantized(self, layer: int) -> bool:
        rc = self._lib.cbkv_layer_is_quantized(self._h, layer)
        check(min(rc, 0))
        return rc == 1

    def export_page_quant(self, layer: int, page: int, stream=None):
        """One int8 page as the reference's Arena::Quant holds it: packed int32 [n_kv, P, d/4] and scale bit
        patterns uint16 [n_kv, P, d/32], for K and for V."""
        kp = np.zeros((self.n_kv_heads, self.page_size, self.head_dim // 4), dtype=np.int32)
        ks = np.zeros((self.n_kv_heads, self.page_size, self.head_dim // 32), dtype=np.uint16)
        vp, vs = np.zeros_like(kp), np.zeros_like(ks)
        sp = _stream_ptr(stream) if torch.cuda.is_available() else 0
        check(self._lib.cbkv_export_page_quant(self._h, layer, page, kp.ctypes.data_as(P), ks.ctypes.data_as(P),
                                               vp.ctypes.data_as(P), vs.ctypes.data_as(P), sp))
        return kp, ks, vp, vs

    def export_page(self, layer: int, page: int, stream=None):
        """One page as the reference lays it out: K and V as [n_kv, page_size, d] uint16 bit patterns."""
        shape = (self.n_kv_heads, self.page_size, self.head_dim)
        k = np.zeros(shape, dtype=np.uint16)
        v = np.zeros(shape, dtype=np.uint16)
        sp = _stream_ptr(stream) if torch.cuda.is_available() else 0
        check(self._lib.cbkv_export_page(self._h, layer, page, k.ctypes.data_as(P), v.ctypes.data_as(P), sp))
        return k, v

    def device_status(self, stream=None) -> int:
        st = C.c_int32(0)
        rc = self._lib.cbkv_device_status(self._h, _stream_ptr(stream), C.byref(st))
        if rc not in (0, -7):
            check(rc)
        return st.value

    def profile_enable(self, on: bool) -> None:
        check(self._lib.cbkv_profile_enable(self._h, 1 if on else 0))

    def profile_read(self):
        ms, n = C.c_double(0), C.c_int64(0)
        check(self._lib.cbkv_profile_read(self._h, C.byref(ms), C.byref(n)))
        return ms.value, n.value

    def set_decode_tuning(self, ctas_per_sm: int = 0, stages: int = 0, consumers: int = 0, max_ctas: int = 0,
                          overlap_launches: bool = True) -> None:
        check(self._lib.cbkv_set_decode_tuning(self._h, ctas_per_sm, stages, consumers, max_ctas,
                                               1 if overlap_launches else 0))

    def set_host_route(self, direct: bool) -> None:
        """attention_host_async on decode steps: True (default) = the kernel waits for a flag written behind its
        inputs, False = the compute stream waits for the input copies' event before every kernel."""
        check(self._lib.cbkv_set_host_route(self._h, 1 if direct else 0))

    def set_chunk_split(self, max_parts: int) -> None:
        """Two-tile chunk kernel: most K/V slices per item of a launch's last, mostly empty wave (1 = never cut)."""
        check(self._lib.cbkv_set_chunk_split(self._h, max_parts))

    def set_chunk_kernel(self, mode: int) -> None:
        """0 = library's choice, 1 = mma.sync chunk kernel, 2 = tcgen05/TMEM kernel (one query tile per
        CTA), 3 = tcgen05/TMEM kernel with two query tiles per CTA (head_dim 128); int8 layers are read
        through a float copy made per layer and step, except in mode 4 = as 3 with the int8 records
        converted inside the kernel (slower so far)."""
        check(self._lib.cbkv_set_chunk_kernel(self._h, mode))

    def set_decode_split(self, tail_pct: int = -1, min_item: int = -1, max_levels: int = -1) -> None:
        """How a CTA's share of a decode launch is cut into a head item and dynamically claimed tail items
        (percent of the share, smallest item in pages with 0 = no tail, levels); negative = keep."""
        check(self._lib.cbkv_set_decode_split(self._h, tail_pct, min_item, max_levels))

    def debug_set_wait_limit(self, wait_us: int = 0, fault_tile: int = -1) -> None:
        """Test hook: limit of the decode kernel's bounded waits, and a tile of CTA 0 whose copy is withheld."""
        check(self._lib.cbkv_debug_set_wait_limit(self._h, wait_us, fault_tile))

    def debug_decode_plan(self, window: int, n_ctas: int, tail_pct: int = -1, min_item: int = -1) -> dict:
        """The decode work split of the step in flight (host only): counts, `segs` [n_segs + 1, 8] and
        `items` [n_items, 4] in claim order (see include/combs_kv.h for the columns)."""
        cap = 1 << 20
        buf = (C.c_int32 * cap)()
        n = self._lib.cbkv_debug_decode_plan(self._h, window, n_ctas, tail_pct, min_item, buf, cap)
        if n < 0 or n > cap:
            raise CbkvError(-6, "no step in flight or plan too large")
        a = np.frombuffer(buf, dtype=np.int32, count=n).copy()
        n_ctas, n_items, n_segs, n_units, n_parts, levels = (int(x) for x in a[:6])
        segs = a[6:6 + (n_segs + 1) * 8].reshape(n_segs + 1, 8)
        items = a[6 + (n_segs + 1) * 8:].reshape(n_items, 4)
        return {"n_ctas": n_ctas, "n_items": n_items, "n_segs": n_segs, "n_units": n_units, "n_parts": n_parts,
                "levels": levels, "segs": segs, "items": items}


def static_status(stream: Optional[torch.cuda.Stream] = None) -> int:
    """Status word of the last ``decode_attention_static`` call on the current device (0 = clean); waits for
    the stream, clears the word, allocates nothing."""
    st = C.c_int32(0)
    rc = _lib.load().cbkv_static_status(_stream_ptr(stream), C.byref(st))
    if rc not in (0, -7):
        check(rc)
    return st.value


def decode_attention_static(kv_pages: torch.Tensor, block_tables: torch.Tensor, seq_lens: Sequence[int],
                            n_q_heads: int, n_kv_heads: int, head_dim: int, q: torch.Tensor,
                            out: Optional[torch.Tensor] = None, scale: Optional[float] = None,
                            window: Optional[int] = None, stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    """Decode attention over caller-owned pages without any device allocation inside the library.

    For callers that may not allocate while they run (the GPU's memory belongs to their
    own pool, or the host process forbids late allocations): the kernel's working memory
    is a fixed array in the library, shared by every call on the device, so calls must
    not overlap on the GPU and sizes are capped (128 sequences, 1024 sequence x kv-head
    pairs).  ``kv_pages`` is one layer ``[num_pages, n_kv, 2, 2, 8, head_dim]`` (slot half, K/V, slot in half),
    ``block_tables`` int32 ``[n_seqs, stride]`` on the device, ``seq_lens`` host integers
    (cached tokens including the one being decoded), ``q``/``out`` ``[n_seqs, n_q, head_dim]``.
    Pass ``out`` to keep even the output allocation on the caller's side.
    """
    lib = _lib.load()
    n = len(seq_lens)
    if out is None:
        out = torch.empty_like(q)
    lens = (C.c_int32 * n)(*[int(x) for x in seq_lens])
    if block_tables.dtype != torch.int32 or not block_tables.is_contiguous() or not kv_pages.is_contiguous():
        raise CbkvError(-4, "block_tables must be contiguous int32 and kv_pages contiguous")
    check(lib.cbkv_decode_attention_static(
        kv_pages.data_ptr(), kv_pages.shape[0], block_tables.data_ptr(), block_tables.shape[1], lens, n,
        n_q_heads, n_kv_heads, head_dim, _DTYPES[kv_pages.dtype], q.data_ptr(), out.data_ptr(),
        float(head_dim ** -0.5 if scale is None else scale), 0 if window is None else int(window), _stream_ptr(stream)))
    return out


def launch_count() -> int:
    """Kernel launches issued by the library in this process."""
    return _lib.load().cbkv_launch_count()


class PagedKVCache:
    """The reference's single-sequence cache (kv.rs:477-855) over a private arena.

    ``attention_opts(layer, q, k, v, pos, scale, window)`` takes q ``[1, n_q, seq, d]``
    and k/v ``[1, n_kv, seq, d]`` CUDA tensors and returns ``[1, n_q, seq, d]``.
    Sliding layers live in pages here and the window is applied as a mask (the
    "masked global" the reference proves equivalent, kv.rs:996-1030), so
    ``pages_used`` counts them and ``layers_sliding`` is always 0.
    """

    def __init__(self, num_layers: int, config: CacheConfig, n_q_heads: int, n_kv_heads: int, head_dim: int,
                 windows: Optional[Sequence[Optional[int]]] = None, dtype: torch.dtype = torch.float16,
                 device: int = 0):
        if config.kind is not CacheKind.Paged:
            raise NotImplementedError("only CacheKind.Paged exists on this path (the cat-per-step baseline is the oracle's)")
        self.config = config
        self.arena = KVArena(num_layers, n_q_heads, n_kv_heads, head_dim, config.max_seq_len, config.page_size,
                             0, windows, dtype, device, quantize_kv=config.quantize_kv)
        self.seq = self.arena.new_seq()

    @classmethod
    def new_with_windows(cls, num_layers, config, windows, **geom) -> "PagedKVCache":  # kv.rs:508-527
        return cls(num_layers, config, windows=windows, **geom)

    def attention(self, layer, q, k, v, pos, scale):  # kv.rs:100-110
        return self.attention_opts(layer, q, k, v, pos, scale, None)

    def attention_opts(self, layer: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, pos: int, scale: float,
                       window: Optional[int] = None) -> torch.Tensor:
        seq = k.shape[-2]
        if layer == 0:  # layer 0 advances the sequence, kv.rs:670-678
            self.arena.begin_step([self.seq], [seq], [pos])
        elif pos + seq != self.seq.seq_len():
            raise CbkvError(-1, "paged cache expects dense contiguous appends (pos == seq_len)")
        return self.arena.attention(layer, q.contiguous(), k.contiguous(), v.contiguous(), scale, window).view(q.shape)

    def seq_len(self) -> int:
        return self.seq.seq_len()

    def popn(self, n: int) -> int:
        return self.seq.popn(n)

    def reset(self) -> None:
        self.seq.reset()

    def pages_used(self) -> int:
        return self.seq.pages_used()

    def num_free_pages(self) -> int:
        return self.arena.num_free_pages()

    def page_stats(self) -> PageStats:
        return self.seq.page_stats()
