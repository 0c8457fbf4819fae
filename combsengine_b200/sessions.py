"""Session table and rollback helpers over a ``KVArena``: host mirror of the reference's
``SessionSet`` and of the two places its runtime rolls the cache back
(combs-runtime/src/engine.rs:266-314, 1257-1287, 1476-1493, 1541-1568).  A thin ctypes layer: the
logic lives in the library (csrc/sessions.cpp)."""
from __future__ import annotations

import ctypes as C
import json
from typing import Optional, Sequence, Tuple

import numpy as np

from . import _lib
from ._lib import check
from .kv import KVArena, PagedSeq

MAX_SESSIONS = 4  # engine.rs:243


def _u32(tokens) -> np.ndarray:
    return np.ascontiguousarray(tokens, dtype=np.uint32)


class SessionSet:
    def __init__(self, arena: KVArena, max_sessions: int = MAX_SESSIONS):
        self.arena = arena
        self._lib = _lib.load()
        h = C.c_void_p()
        check(self._lib.cbkv_sessions_create(arena._h, max_sessions, C.byref(h)))
        self._h = h.value
        self._held: dict[str, PagedSeq] = {}   # key -> wrapper of the sequence the table owns

    @staticmethod
    def _drop(w: PagedSeq) -> None:
        """The library destroyed this sequence: disarm its wrapper."""
        w._h = None
        w.arena._seqs.discard(w)

    def close(self) -> None:
        if getattr(self, "_h", None):
            for w in self._held.values():
                self._drop(w)
            self._held.clear()
            self._lib.cbkv_sessions_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def acquire(self, key: Optional[str], prompt: Sequence[int], reuse: bool = True) -> Tuple[PagedSeq, int]:
        """engine.rs:1257-1287 -> (sequence, lcp): prefill starts at token ``lcp`` of the prompt."""
        key = key or ""
        p = _u32(prompt)
        seq, lcp = C.c_void_p(), C.c_int64(0)
        check(self._lib.cbkv_sessions_acquire(self._h, key.encode(), p.ctypes.data_as(C.c_void_p), len(p),
                                              1 if reuse else 0, C.byref(seq), C.byref(lcp)))
        w = self._held.pop(key, None) if reuse else None
        if w is not None and w._h != seq.value:   # the old cache could not be reused and was dropped
            self._drop(w)
            w = None
        return (w or PagedSeq(self.arena, seq.value)), lcp.value

    def release(self, key: Optional[str], seq: PagedSeq, history: Sequence[int], reuse: bool = True) -> None:
        """engine.rs:1541-1568 + SessionSet::put (:296-313)."""
        key = key or ""
        h = _u32(history)
        check(self._lib.cbkv_sessions_release(self._h, key.encode(), seq._h, h.ctypes.data_as(C.c_void_p), len(h),
                                              1 if reuse else 0))
        if not reuse:
            self._drop(seq)
            return
        old = self._held.get(key)
        if old is not None and old is not seq:
            self._drop(old)
        self._held[key] = seq
        for k in [k for k in self._held if self._lib.cbkv_sessions_history_len(self._h, k.encode()) < 0]:
            self._drop(self._held.pop(k))     # evicted as least recently used

    def clear_all(self) -> int:
        n = C.c_int64(0)
        check(self._lib.cbkv_sessions_clear(self._h, C.byref(n)))
        for w in self._held.values():
            self._drop(w)
        self._held.clear()
        return n.value

    def __len__(self) -> int:
        return self._lib.cbkv_sessions_count(self._h)

    @property
    def evictions(self) -> int:
        return self._lib.cbkv_sessions_evictions(self._h)

    def history_len(self, key: Optional[str]) -> Optional[int]:
        n = self._lib.cbkv_sessions_history_len(self._h, (key or "").encode())
        return None if n < 0 else n

    def stats_json(self) -> str:
        """The "kv" object of GET /v1/stats (serve.rs:146-166,197-208)."""
        n = self._lib.cbkv_sessions_stats_json(self._h, None, 0)
        buf = C.create_string_buffer(n + 1)
        self._lib.cbkv_sessions_stats_json(self._h, buf, n + 1)
        return buf.value.decode()

    def stats(self) -> dict:
        return json.loads(self.stats_json())


def spec_verify_rollback(seq: PagedSeq, draft: Sequence[int], argmax: Sequence[int]) -> Tuple[int, int]:
    """engine.rs:1476-1493 -> (accepted, correction); the rejected tail leaves the cache."""
    d, a = _u32(draft), _u32(argmax)
    assert len(a) == len(d) + 1, "argmax has one row per fed token: next + the draft"
    acc, corr = C.c_int32(0), C.c_uint32(0)
    check(seq.arena._lib.cbkv_spec_verify_rollback(seq._h, d.ctypes.data_as(C.c_void_p), a.ctypes.data_as(C.c_void_p), len(d),
                                                   C.byref(acc), C.byref(corr)))
    return acc.value, corr.value
