"""B200-native paged KV cache + attention: the KVCache path of CombsEngine.

The compute lives in ``libcombskv.so`` (hand-written CUDA for sm_100a behind the C
ABI of ``include/combs_kv.h``); this package is the host-side mirror of the
reference's operator surface (``combs-models/src/kv.rs``).
"""
from .kv import (CacheConfig, CacheKind, KVArena, PagedKVCache, PagedSeq, PageStats, CbkvError)
from .rope import QKNorm, RopeScaling, RotaryEmbedding, attention_rope, rope_append
from .sessions import SessionSet, spec_verify_rollback

__all__ = ["CacheConfig", "CacheKind", "KVArena", "PagedKVCache", "PagedSeq", "PageStats", "CbkvError",
           "QKNorm", "RopeScaling", "RotaryEmbedding", "attention_rope", "rope_append", "SessionSet", "spec_verify_rollback"]
