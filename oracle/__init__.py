"""CPU oracle for the paged KV cache path — TEST INFRASTRUCTURE ONLY.

ctypes wrapper over ``kv_oracle.c`` (the C restatement of the reference's
``engine/core/combs-models/src/kv.rs``).  Only the tests, the smoke check and
the CPU-baseline leg of the benchmark may import this package; the product
package ``combsengine_b200`` never does.

Floating-point parity is unpinned in the golden-vector sense (the reference
stores no attention outputs); integer/state behaviour is pinned by the
reference's own known-answer tests.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIBS: dict[str, C.CDLL] = {}

I64 = C.c_int64
P = C.c_void_p


def build(force: bool = False) -> None:
    """Compile the oracle (gcc, a few seconds)."""
    out = os.path.join(_HERE, "_build")
    if not force and all(os.path.exists(os.path.join(out, f"liborc_{k}.so")) for k in ("f32", "f16")):
        src = max(os.path.getmtime(os.path.join(_HERE, f)) for f in ("kv_oracle.c", "rope_oracle.c", "Makefile"))
        if all(os.path.getmtime(os.path.join(out, f"liborc_{k}.so")) >= src for k in ("f32", "f16")):
            return
    subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)


def _lib(kind: str) -> C.CDLL:
    if kind in _LIBS:
        return _LIBS[kind]
    path = os.path.join(_HERE, "_build", f"liborc_{kind}.so")
    if not os.path.exists(path):
        build()
    lib = C.CDLL(path)
    lib.orc_last_error.restype = C.c_char_p
    lib.orc_arena_new.restype = P
    lib.orc_arena_new.argtypes = [C.c_int, C.c_int, C.c_int, I64, C.c_int, I64, P, C.c_int]
    lib.orc_arena_free.argtypes = [P]
    lib.orc_set_free_list.argtypes = [P, P, I64]
    lib.orc_seq_new.restype = P
    lib.orc_seq_new.argtypes = [P]
    lib.orc_seq_free.argtypes = [P]
    lib.orc_seq_fork_prefix.restype = P
    lib.orc_seq_fork_prefix.argtypes = [P, I64]
    lib.orc_grow.argtypes = [P, I64]
    lib.orc_begin.argtypes = [P, I64, I64]
    for name in ("orc_layer", "orc_attention", "orc_contig_attention"):
        getattr(lib, name).argtypes = [P, C.c_int, P, P, P, P, C.c_int, I64, I64, C.c_double, I64]
    lib.orc_append_only.argtypes = [P, C.c_int, P, P, I64, I64]
    lib.orc_popn.restype = I64
    lib.orc_popn.argtypes = [P, I64]
    lib.orc_reset.argtypes = [P]
    for name in ("orc_seq_len", "orc_pages_used", "orc_num_free_pages", "orc_contig_seq_len"):
        getattr(lib, name).restype = I64
        getattr(lib, name).argtypes = [P]
    lib.orc_page_stats.argtypes = [P, P]
    lib.orc_export_block_table.restype = I64
    lib.orc_export_block_table.argtypes = [P, P, I64]
    lib.orc_export_free_list.restype = I64
    lib.orc_export_free_list.argtypes = [P, P, I64]
    lib.orc_export_page.argtypes = [P, C.c_int, I64, P, P]
    lib.orc_page_refcount.restype = C.c_int32
    lib.orc_page_refcount.argtypes = [P, I64]
    lib.orc_contig_new.restype = P
    lib.orc_contig_new.argtypes = [C.c_int, C.c_int, C.c_int]
    lib.orc_contig_reset.argtypes = [P]
    lib.orc_contig_free.argtypes = [P]
    lib.orc_batch_begin.argtypes = [P, P, C.c_int]
    lib.orc_batch_layer.argtypes = [P, P, C.c_int, C.c_int, P, P, P, P, C.c_int, C.c_double, I64]
    _LIBS[kind] = lib
    return lib


def set_threads(n: int, kind: str = "f16") -> int:
    """OpenMP threads used by the batch driver; returns the number in effect."""
    lib = _lib(kind)
    lib.orc_set_threads.argtypes = [C.c_int]
    lib.orc_set_threads.restype = C.c_int
    return lib.orc_set_threads(int(n))


class OracleError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(msg)
        self.code = code


PAGE_STATS_FIELDS = ("pages_used", "pages_free", "num_pages", "page_size", "seq_len",
                     "layers_materialized", "layers_total", "layers_sliding")


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(P)


class OracleArena:
    """Arena + allocator shared by the sequences created from it."""

    def __init__(self, layers: int, n_kv: int, head_dim: int, max_seq_len: int, page_size: int = 16,
                 num_pages: int = 0, windows=None, rolling: bool = True, dtype: str = "f16", quantize_kv: bool = False):
        self.kind = dtype
        self.np_dtype = np.float16 if dtype == "f16" else np.float32
        self.lib = _lib(dtype)
        self.layers, self.n_kv, self.d, self.page_size = layers, n_kv, head_dim, page_size
        w = None
        if windows is not None:
            assert len(windows) == layers, "one window entry per layer"
            w = np.asarray([0 if x is None else int(x) for x in windows], dtype=np.int64)
        self.h = self.lib.orc_arena_new(layers, n_kv, head_dim, max_seq_len, page_size, num_pages,
                                        _ptr(w) if w is not None else None, 1 if rolling else 0)
        if not self.h:
            raise OracleError(-4, self.lib.orc_last_error().decode())
        self.num_pages = num_pages if num_pages > 0 else -(-max_seq_len // page_size)
        self._seqs = []
        if quantize_kv:
            self.lib.orc_arena_set_quantize.argtypes = [P, C.c_int]
            self.lib.orc_arena_set_quantize(self.h, 1)

    def __del__(self):
        try:
            for s in list(self._seqs):
                s.close()
            if self.h:
                self.lib.orc_arena_free(self.h)
                self.h = None
        except Exception:
            pass

    def set_free_list(self, ids) -> None:
        a = np.ascontiguousarray(ids, dtype=np.int64)
        rc = self.lib.orc_set_free_list(self.h, _ptr(a), len(a))
        if rc:
            raise OracleError(rc, self.lib.orc_last_error().decode())

    def new_seq(self) -> "OracleSeq":
        return OracleSeq(self, self.lib.orc_seq_new(self.h))

    def num_free_pages(self) -> int:
        return self.lib.orc_num_free_pages(self.h)

    def free_list(self) -> np.ndarray:
        out = np.zeros(self.num_pages, dtype=np.int64)
        n = self.lib.orc_export_free_list(self.h, _ptr(out), len(out))
        return out[:n]

    def page_quant(self, layer: int, page: int):
        """Arena::Quant contents of one page (kv.rs:464-475): packed int32 [n_kv, P, d/4] and scales
        [n_kv, P, d/32] for K and for V."""
        kp = np.zeros((self.n_kv, self.page_size, self.d // 4), dtype=np.int32)
        ks = np.zeros((self.n_kv, self.page_size, self.d // 32), dtype=self.np_dtype)
        vp, vs = np.zeros_like(kp), np.zeros_like(ks)
        self.lib.orc_export_page_quant.argtypes = [P, C.c_int, I64, P, P, P, P]
        self.lib.orc_export_page_quant(self.h, layer, page, _ptr(kp), _ptr(ks), _ptr(vp), _ptr(vs))
        return kp, ks, vp, vs

    def page(self, layer: int, page: int):
        k = np.zeros((self.n_kv, self.page_size, self.d), dtype=self.np_dtype)
        v = np.zeros_like(k)
        self.lib.orc_export_page(self.h, layer, page, _ptr(k), _ptr(v))
        return k, v

    def refcount(self, page: int) -> int:
        return self.lib.orc_page_refcount(self.h, page)

    # batch driver (timed CPU baseline): packed per-sequence [H, s_b, d] blocks
    def batch_begin(self, seqs, new_tokens) -> None:
        hs = (P * len(seqs))(*[s.h for s in seqs])
        nt = np.ascontiguousarray(new_tokens, dtype=np.int64)
        rc = self.lib.orc_batch_begin(hs, _ptr(nt), len(seqs))
        if rc:
            raise OracleError(rc, self.lib.orc_last_error().decode())

    def batch_layer(self, seqs, new_tokens, layer, q, k, v, n_q, scale, window=None) -> np.ndarray:
        hs = (P * len(seqs))(*[s.h for s in seqs])
        nt = np.ascontiguousarray(new_tokens, dtype=np.int64)
        q = np.ascontiguousarray(q, dtype=self.np_dtype)
        k = np.ascontiguousarray(k, dtype=self.np_dtype)
        v = np.ascontiguousarray(v, dtype=self.np_dtype)
        out = np.empty_like(q)
        rc = self.lib.orc_batch_layer(hs, _ptr(nt), len(seqs), layer, _ptr(q), _ptr(k), _ptr(v), _ptr(out),
                                      n_q, float(scale), 0 if window is None else int(window))
        if rc:
            raise OracleError(rc, self.lib.orc_last_error().decode())
        return out


class OracleSeq:
    """One sequence; alone in a fresh arena it is the reference's PagedKVCache."""

    def __init__(self, arena: OracleArena, handle):
        self.arena, self.lib, self.h = arena, arena.lib, handle
        arena._seqs.append(self)

    def close(self):
        if self.h:
            self.lib.orc_seq_free(self.h)
            self.h = None
            self.arena._seqs.remove(self)

    def _check(self, rc):
        if rc:
            raise OracleError(rc, self.lib.orc_last_error().decode())

    def _call(self, fn, layer, q, k, v, pos, scale, window):
        dt = self.arena.np_dtype
        q = np.ascontiguousarray(q, dtype=dt)
        k = np.ascontiguousarray(k, dtype=dt)
        v = np.ascontiguousarray(v, dtype=dt)
        lead = q.shape[:-3]
        n_q, seq, d = q.shape[-3:]
        assert k.shape[-3:] == (self.arena.n_kv, seq, d) and v.shape == k.shape
        out = np.empty_like(q)
        self._check(fn(self.h, layer, _ptr(q), _ptr(k), _ptr(v), _ptr(out), n_q, seq, pos, float(scale),
                       0 if window is None else int(window)))
        return out.reshape(lead + (n_q, seq, d))

    def attention_opts(self, layer, q, k, v, pos, scale, window=None):
        """q [1,n_q,seq,d] (or [n_q,seq,d]); k, v [1,n_kv,seq,d]; returns q's shape."""
        return self._call(self.lib.orc_attention, layer, q, k, v, pos, scale, window)

    def attention(self, layer, q, k, v, pos, scale):
        return self.attention_opts(layer, q, k, v, pos, scale, None)

    def begin(self, pos, seq):
        self._check(self.lib.orc_begin(self.h, pos, seq))

    def layer(self, layer, q, k, v, pos, scale, window=None):
        return self._call(self.lib.orc_layer, layer, q, k, v, pos, scale, window)

    def append_only(self, layer, k, v, pos):
        """Fill rows without attending (benchmark set-up); k, v [n_kv, seq, d]."""
        dt = self.arena.np_dtype
        k = np.ascontiguousarray(k, dtype=dt)
        v = np.ascontiguousarray(v, dtype=dt)
        self._check(self.lib.orc_append_only(self.h, layer, _ptr(k), _ptr(v), k.shape[-2], pos))

    def grow(self, total):
        self._check(self.lib.orc_grow(self.h, total))

    def fork_prefix(self, n_tokens) -> "OracleSeq":
        h = self.lib.orc_seq_fork_prefix(self.h, n_tokens)
        if not h:
            raise OracleError(-4, self.lib.orc_last_error().decode())
        return OracleSeq(self.arena, h)

    def popn(self, n) -> int:
        return self.lib.orc_popn(self.h, n)

    def reset(self):
        self.lib.orc_reset(self.h)

    def seq_len(self) -> int:
        return self.lib.orc_seq_len(self.h)

    def pages_used(self) -> int:
        return self.lib.orc_pages_used(self.h)

    def num_free_pages(self) -> int:
        return self.arena.num_free_pages()

    def page_stats(self) -> dict:
        out = np.zeros(8, dtype=np.int64)
        self.lib.orc_page_stats(self.h, _ptr(out))
        return dict(zip(PAGE_STATS_FIELDS, (int(x) for x in out)))

    def block_table(self) -> np.ndarray:
        out = np.zeros(max(1, self.pages_used()), dtype=np.int64)
        n = self.lib.orc_export_block_table(self.h, _ptr(out), len(out))
        return out[:n]


class OracleContiguous:
    """ContiguousKVCache (kv.rs:360-415), the reference's cross-validation baseline."""

    def __init__(self, layers, n_kv, head_dim, dtype="f32"):
        self.lib = _lib(dtype)
        self.np_dtype = np.float16 if dtype == "f16" else np.float32
        self.n_kv = n_kv
        self.h = self.lib.orc_contig_new(layers, n_kv, head_dim)

    def __del__(self):
        try:
            if self.h:
                self.lib.orc_contig_free(self.h)
                self.h = None
        except Exception:
            pass

    def attention_opts(self, layer, q, k, v, pos, scale, window=None):
        dt = self.np_dtype
        q = np.ascontiguousarray(q, dtype=dt)
        k = np.ascontiguousarray(k, dtype=dt)
        v = np.ascontiguousarray(v, dtype=dt)
        n_q, seq, d = q.shape[-3:]
        out = np.empty_like(q)
        rc = self.lib.orc_contig_attention(self.h, layer, _ptr(q), _ptr(k), _ptr(v), _ptr(out), n_q, seq, pos,
                                           float(scale), 0 if window is None else int(window))
        assert rc == 0
        return out

    def attention(self, layer, q, k, v, pos, scale):
        return self.attention_opts(layer, q, k, v, pos, scale, None)

    def seq_len(self):
        return self.lib.orc_contig_seq_len(self.h)

    def reset(self):
        self.lib.orc_contig_reset(self.h)

    def popn(self, n):  # KVCache default, kv.rs:133-136
        return 0


# ---------------------------------------------------------------------------------------------
# Rotary embedding and QK norm (rope_oracle.c): the step right before the cache.
ROPE_KINDS = {"none": 0, "linear": 1, "llama3": 2, "yarn": 3, "longrope": 4}


def rope_inv_freq(head_dim: int, theta: float, scaling: dict | None = None):
    """``scaled_inv_freq`` (rope.rs:31-125) -> (inv_freq f64[head_dim/2], mscale)."""
    s = dict(scaling or {})
    kind = ROPE_KINDS[s.get("kind", "none")]
    lib = _lib("f32")
    lib.orc_rope_inv_freq.argtypes = [C.c_int, C.c_double, C.c_int, C.c_double, C.c_double, C.c_double, C.c_double,
                                      C.c_double, I64, C.c_double, P, C.c_int, P, P]
    inv = np.zeros(head_dim // 2, dtype=np.float64)
    ms = C.c_double(0.0)
    short = np.ascontiguousarray(s.get("short_factor", []), dtype=np.float64)
    af = s.get("attention_factor")
    rc = lib.orc_rope_inv_freq(head_dim, float(theta), kind, float(s.get("factor", 1.0)),
                               float(s.get("low_freq_factor", 1.0)), float(s.get("high_freq_factor", 1.0)),
                               float(s.get("beta_fast", 32.0)), float(s.get("beta_slow", 1.0)),
                               int(s.get("original_max_position_embeddings", 0)),
                               float("nan") if af is None else float(af),
                               _ptr(short) if len(short) else None, len(short), _ptr(inv), C.byref(ms))
    if rc:
        raise OracleError(rc, "unknown rope scaling kind")
    return inv, ms.value


def rope_tables(head_dim: int, theta: float, max_position: int, scaling: dict | None = None):
    """``build_tables_scaled`` (rope.rs:129-151) -> (cos, sin) f32 [max_position, head_dim]."""
    inv, ms = rope_inv_freq(head_dim, theta, scaling)
    lib = _lib("f32")
    lib.orc_rope_tables.argtypes = [C.c_int, I64, P, C.c_double, P, P]
    cos = np.zeros((max_position, head_dim), dtype=np.float32)
    sin = np.zeros_like(cos)
    lib.orc_rope_tables(head_dim, max_position, _ptr(inv), ms, _ptr(cos), _ptr(sin))
    return cos, sin


def rope_apply(x: np.ndarray, pos: int, cos: np.ndarray, sin: np.ndarray) -> np.ndarray:
    """``RotaryEmbedding::apply`` (rope.rs:180-204) on x [heads, seq, d] (f16 or f32)."""
    kind = "f16" if x.dtype == np.float16 else "f32"
    lib = _lib(kind)
    lib.orc_rope_apply.argtypes = [P, C.c_int, I64, C.c_int, I64, P, P]
    out = np.ascontiguousarray(x).copy()
    heads, seq, d = out.shape
    assert cos.shape[1] == d and pos + seq <= cos.shape[0], "position outside the rope table"
    lib.orc_rope_apply(_ptr(out), heads, seq, d, int(pos), _ptr(np.ascontiguousarray(cos)), _ptr(np.ascontiguousarray(sin)))
    return out


def rms_norm(x: np.ndarray, w: np.ndarray, eps: float, gemma: bool = False) -> np.ndarray:
    """``rms_norm`` / ``gemma_rms_norm`` (norm.rs:11-39) over the last dim."""
    kind = "f16" if x.dtype == np.float16 else "f32"
    lib = _lib(kind)
    lib.orc_rms_norm.argtypes = [P, I64, C.c_int, P, C.c_double, C.c_int]
    out = np.ascontiguousarray(x).copy()
    d = out.shape[-1]
    w = np.ascontiguousarray(w, dtype=x.dtype)
    lib.orc_rms_norm(_ptr(out), out.size // d, d, _ptr(w), float(eps), 1 if gemma else 0)
    return out


# ---------------------------------------------------------------------------------------------
# int8 KV pages (kv.rs:271-358)
def kv_quantize(x: np.ndarray):
    """``kv_quantize`` on x [..., d] (d % 32 == 0) -> (packed int32 [..., d/4], scales [..., d/32])."""
    kind = "f16" if x.dtype == np.float16 else "f32"
    lib = _lib(kind)
    lib.orc_kv_quantize.argtypes = [P, I64, C.c_int, P, P]
    x = np.ascontiguousarray(x)
    d = x.shape[-1]
    packed = np.zeros(x.shape[:-1] + (d // 4,), dtype=np.int32)
    scales = np.zeros(x.shape[:-1] + (d // 32,), dtype=x.dtype)
    lib.orc_kv_quantize(_ptr(x), x.size // d, d, _ptr(packed), _ptr(scales))
    return packed, scales


def kv_dequantize(packed: np.ndarray, scales: np.ndarray, d: int) -> np.ndarray:
    """``kv_dequantize`` -> [..., d] in the dtype of ``scales``."""
    kind = "f16" if scales.dtype == np.float16 else "f32"
    lib = _lib(kind)
    lib.orc_kv_dequantize.argtypes = [P, P, I64, C.c_int, P]
    packed, scales = np.ascontiguousarray(packed), np.ascontiguousarray(scales)
    out = np.zeros(packed.shape[:-1] + (d,), dtype=scales.dtype)
    lib.orc_kv_dequantize(_ptr(packed), _ptr(scales), out.size // d, d, _ptr(out))
    return out
