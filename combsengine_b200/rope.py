"""Rotary embedding and QK norm fused into the append: host mirror of the reference types.

``RopeScaling`` / ``RotaryEmbedding`` carry the names and arguments of
``combs_formats::RopeScaling`` and ``combs-models/src/rope.rs``; the tables are built by the
library's host code and live on the arena's device, and ``KVArena``-level calls
(`rope_append`, `attention_rope`) run the fused kernel.  No fallback: every call goes through
``libcombskv.so``.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np
import torch

from . import _lib
from ._lib import CbkvError, check
from .kv import KVArena, _stream_ptr

_KINDS = {"none": 0, "linear": 1, "llama3": 2, "yarn": 3, "longrope": 4}


@dataclass
class RopeScaling:
    """combs_formats::RopeScaling: None | Linear | Llama3 | Yarn | LongRope (rope.rs:36-124)."""
    kind: str = "none"
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 1.0
    beta_fast: float = 32.0
    beta_slow: float = 1.0
    original_max_position_embeddings: int = 0
    attention_factor: Optional[float] = None
    short_factor: Sequence[float] = field(default_factory=list)

    @classmethod
    def from_dict(cls, d: Optional[dict]) -> "RopeScaling":
        return cls(**(d or {}))


def _config(head_dim: int, theta: float, max_position: int, scaling: Optional[RopeScaling]):
    s = scaling or RopeScaling()
    if s.kind not in _KINDS:
        raise CbkvError(-4, f"unknown rope scaling {s.kind!r}")
    short = (C.c_double * max(1, len(s.short_factor)))(*[float(x) for x in s.short_factor])
    cfg = _lib.cbkv_rope_config(
        head_dim=head_dim, scaling=_KINDS[s.kind], theta=float(theta), max_position=int(max_position),
        factor=float(s.factor), low_freq_factor=float(s.low_freq_factor), high_freq_factor=float(s.high_freq_factor),
        beta_fast=float(s.beta_fast), beta_slow=float(s.beta_slow),
        original_max_position=int(s.original_max_position_embeddings),
        has_attention_factor=0 if s.attention_factor is None else 1,
        attention_factor=0.0 if s.attention_factor is None else float(s.attention_factor),
        short_factor=C.cast(short, C.POINTER(C.c_double)), n_short_factor=len(s.short_factor))
    return cfg, short  # keep `short` alive with the config


def scaled_inv_freq(head_dim: int, theta: float, scaling: Optional[RopeScaling] = None):
    """rope.rs:31-125 -> (inv_freq float64[head_dim/2], mscale).  Host only."""
    cfg, _keep = _config(head_dim, theta, 1, scaling)
    inv = np.zeros(head_dim // 2, dtype=np.float64)
    ms = C.c_double(0.0)
    check(_lib.load().cbkv_rope_inv_freq_host(C.byref(cfg), inv.ctypes.data_as(C.c_void_p), C.byref(ms)))
    return inv, ms.value


def build_tables_scaled(head_dim: int, theta: float, max_position: int, scaling: Optional[RopeScaling] = None):
    """rope.rs:129-151 -> (cos, sin) float32 [max_position, head_dim].  Host only."""
    cfg, _keep = _config(head_dim, theta, max_position, scaling)
    cos = np.zeros((max_position, head_dim), dtype=np.float32)
    sin = np.zeros_like(cos)
    check(_lib.load().cbkv_rope_tables_host(C.byref(cfg), cos.ctypes.data_as(C.c_void_p), sin.ctypes.data_as(C.c_void_p)))
    return cos, sin


def build_tables(head_dim: int, theta: float, max_position: int):
    """rope.rs:22-28."""
    return build_tables_scaled(head_dim, theta, max_position, None)


class RotaryEmbedding:
    """rope.rs:15-18,153-177: tables on the arena's device, in the arena's element type."""

    def __init__(self, arena: KVArena, theta: float, max_position: int, scaling: Optional[RopeScaling] = None):
        self.arena = arena
        self._lib = _lib.load()
        cfg, _keep = _config(arena.head_dim, theta, max_position, scaling)
        h = C.c_void_p()
        check(self._lib.cbkv_rope_create(arena._h, C.byref(cfg), C.byref(h)))
        self._h = h.value
        self.max_position = max_position

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.cbkv_rope_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


@dataclass
class QKNorm:
    """Per-head norm weights of a layer (llama.rs:275-281): tensors of head_dim elements on the
    arena's device, either may be None; ``gemma`` selects x̂·(1+w) (norm.rs:33-39)."""
    q_weight: Optional[torch.Tensor]
    k_weight: Optional[torch.Tensor]
    eps: float = 1e-6
    gemma: bool = False

    def _struct(self, arena: KVArena):
        for w in (self.q_weight, self.k_weight):
            if w is not None and not (w.is_cuda and w.is_contiguous() and w.dtype == arena.dtype and w.numel() == arena.head_dim):
                raise CbkvError(-4, "norm weight must be a contiguous CUDA tensor of head_dim elements in the arena's dtype")
        return _lib.cbkv_qk_norm(q_weight=None if self.q_weight is None else self.q_weight.data_ptr(),
                                 k_weight=None if self.k_weight is None else self.k_weight.data_ptr(),
                                 eps=float(self.eps), gemma=1 if self.gemma else 0)


def rope_append(arena: KVArena, layer: int, rope: RotaryEmbedding, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                norm: Optional[QKNorm] = None, q_out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
    """Norm + rotate q (returned), norm + rotate k and copy v into the step's page slots."""
    arena._chk(q, arena.n_q_heads, "q"); arena._chk(k, arena.n_kv_heads, "k"); arena._chk(v, arena.n_kv_heads, "v")
    if q_out is None:
        q_out = torch.empty_like(q)
    ns = norm._struct(arena) if norm is not None else None
    check(arena._lib.cbkv_rope_append(arena._h, layer, rope._h, C.byref(ns) if ns is not None else None, q.data_ptr(),
                                      k.data_ptr(), v.data_ptr(), q_out.data_ptr(), _stream_ptr(stream)))
    return q_out


def attention_rope(arena: KVArena, layer: int, rope: RotaryEmbedding, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                   scale: float, window: Optional[int] = None, norm: Optional[QKNorm] = None,
                   out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
    """llama.rs:275-289 for one layer: QK norm, rotation, append, attention."""
    arena._chk(q, arena.n_q_heads, "q"); arena._chk(k, arena.n_kv_heads, "k"); arena._chk(v, arena.n_kv_heads, "v")
    if out is None:
        out = torch.empty_like(q)
    ns = norm._struct(arena) if norm is not None else None
    check(arena._lib.cbkv_attention_rope(arena._h, layer, rope._h, C.byref(ns) if ns is not None else None, q.data_ptr(),
                                         k.data_ptr(), v.data_ptr(), out.data_ptr(), float(scale),
                                         0 if window is None else int(window), _stream_ptr(stream)))
    return out
