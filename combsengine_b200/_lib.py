"""ctypes binding of libcombskv.so (the C ABI declared in include/combs_kv.h).

There is no fallback: if the CUDA library is missing the import fails, and on a
machine without a B200 every compute call returns an error.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libcombskv.so")

I32, I64, F64, P = C.c_int32, C.c_int64, C.c_double, C.c_void_p


class cbkv_config(C.Structure):
    _fields_ = [
        ("num_layers", I32), ("n_q_heads", I32), ("n_kv_heads", I32), ("head_dim", I32),
        ("page_size", I32), ("dtype", I32), ("max_seq_len", I64), ("num_pages", I64),
        ("layer_windows", C.POINTER(I64)), ("sliding_popn_refuses", I32), ("device", I32),
        ("quantize_kv", I32),
    ]


class cbkv_page_stats_t(C.Structure):
    _fields_ = [(n, I64) for n in ("pages_used", "pages_free", "num_pages", "page_size", "seq_len",
                                   "layers_materialized", "layers_total", "layers_sliding")]


class cbkv_rope_config(C.Structure):
    _fields_ = [
        ("head_dim", I32), ("scaling", I32), ("theta", F64), ("max_position", I64), ("factor", F64),
        ("low_freq_factor", F64), ("high_freq_factor", F64), ("beta_fast", F64), ("beta_slow", F64),
        ("original_max_position", I64), ("has_attention_factor", I32), ("attention_factor", F64),
        ("short_factor", C.POINTER(F64)), ("n_short_factor", I32),
    ]


class cbkv_qk_norm(C.Structure):
    _fields_ = [("q_weight", P), ("k_weight", P), ("eps", F64), ("gemma", I32)]


# name -> (restype, argtypes); every symbol include/combs_kv.h declares
PROTOTYPES = {
    "cbkv_last_error": (C.c_char_p, []),
    "cbkv_arena_create": (I32, [C.POINTER(cbkv_config), C.POINTER(P)]),
    "cbkv_arena_destroy": (I32, [P]),
    "cbkv_set_free_list": (I32, [P, C.POINTER(I64), I64]),
    "cbkv_seq_create": (I32, [P, C.POINTER(P)]),
    "cbkv_seq_destroy": (I32, [P]),
    "cbkv_seq_fork_prefix": (I32, [P, I64, C.POINTER(P)]),
    "cbkv_begin_step": (I32, [P, C.POINTER(P), C.POINTER(I64), C.POINTER(I64), I32, P]),
    "cbkv_append": (I32, [P, I32, P, P, P]),
    "cbkv_paged_attention": (I32, [P, I32, P, P, F64, I64, P]),
    "cbkv_attention": (I32, [P, I32, P, P, P, P, F64, I64, P]),
    "cbkv_attention_host": (I32, [P, I32, P, P, P, P, F64, I64, P]),
    "cbkv_decode_attention_static": (I32, [P, I64, P, I32, C.POINTER(I32), I32, I32, I32, I32, I32, P, P, F64, I64, P]),
    "cbkv_rope_tables_host": (I32, [C.POINTER(cbkv_rope_config), P, P]),
    "cbkv_rope_inv_freq_host": (I32, [C.POINTER(cbkv_rope_config), P, C.POINTER(F64)]),
    "cbkv_rope_create": (I32, [P, C.POINTER(cbkv_rope_config), C.POINTER(P)]),
    "cbkv_rope_destroy": (I32, [P]),
    "cbkv_rope_append": (I32, [P, I32, P, C.POINTER(cbkv_qk_norm), P, P, P, P, P]),
    "cbkv_attention_rope": (I32, [P, I32, P, C.POINTER(cbkv_qk_norm), P, P, P, P, F64, I64, P]),
    "cbkv_sessions_create": (I32, [P, I32, C.POINTER(P)]),
    "cbkv_sessions_destroy": (I32, [P]),
    "cbkv_sessions_acquire": (I32, [P, C.c_char_p, P, I64, I32, C.POINTER(P), C.POINTER(I64)]),
    "cbkv_sessions_release": (I32, [P, C.c_char_p, P, P, I64, I32]),
    "cbkv_sessions_clear": (I32, [P, C.POINTER(I64)]),
    "cbkv_sessions_count": (I64, [P]),
    "cbkv_sessions_evictions": (I64, [P]),
    "cbkv_sessions_history_len": (I64, [P, C.c_char_p]),
    "cbkv_spec_verify_rollback": (I32, [P, P, P, I32, C.POINTER(I32), C.POINTER(C.c_uint32)]),
    "cbkv_sessions_stats_json": (I64, [P, C.c_char_p, I64]),
    "cbkv_attention_host_async": (I32, [P, I32, P, P, P, P, F64, I64, P]),
    "cbkv_host_sync": (I32, [P]),
    "cbkv_host_alloc": (I32, [C.c_size_t, C.POINTER(P)]),
    "cbkv_host_free": (I32, [P]),
    "cbkv_popn": (I32, [P, I64, C.POINTER(I64)]),
    "cbkv_reset": (I32, [P]),
    "cbkv_seq_len": (I64, [P]),
    "cbkv_pages_used": (I64, [P]),
    "cbkv_num_free_pages": (I64, [P]),
    "cbkv_page_stats": (I32, [P, C.POINTER(cbkv_page_stats_t)]),
    "cbkv_page_bytes": (I64, [P]),
    "cbkv_export_block_table": (I64, [P, C.POINTER(I64), I64]),
    "cbkv_export_free_list": (I64, [P, C.POINTER(I64), I64]),
    "cbkv_export_page": (I32, [P, I32, I64, P, P, P]),
    "cbkv_export_page_quant": (I32, [P, I32, I64, P, P, P, P, P]),
    "cbkv_layer_is_quantized": (I32, [P, I32]),
    "cbkv_page_refcount": (I32, [P, I64]),
    "cbkv_device_status": (I32, [P, P, C.POINTER(I32)]),
    "cbkv_launch_count": (I64, []),
    "cbkv_profile_enable": (I32, [P, I32]),
    "cbkv_profile_read": (I32, [P, C.POINTER(F64), C.POINTER(I64)]),
    "cbkv_set_decode_tuning": (I32, [P, I32, I32, I32, I32, I32]),
    "cbkv_set_chunk_kernel": (I32, [P, I32]),
    "cbkv_set_host_route": (I32, [P, I32]),
    "cbkv_set_chunk_split": (I32, [P, I32]),
    "cbkv_debug_begin_step_host": (I32, [P, C.POINTER(P), C.POINTER(I64), C.POINTER(I64), I32]),
    "cbkv_debug_decode_plan": (I64, [P, I64, I32, I32, I32, C.POINTER(I32), I64]),
    "cbkv_set_decode_split": (I32, [P, I32, I32, I32]),
    "cbkv_debug_set_wait_limit": (I32, [P, I64, I32]),
    "cbkv_static_status": (I32, [P, C.POINTER(I32)]),
    "cbkv_debug_raise": (I32, [I32]),
}

_lib = None


def use_measure_build() -> None:
    """Load the measurement flavour (python -m combsengine_b200._build --measure) instead of the
    product library; must be called before the first load()."""
    global LIB_PATH
    if _lib is not None:
        raise RuntimeError("the library is already loaded")
    LIB_PATH = os.path.join(HERE, "libcombskv_measure.so")


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m combsengine_b200._build` "
            "(nvcc, sm_100a). There is no CPU or PyTorch fallback for this path.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError if the library does not export it
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


class CbkvError(RuntimeError):
    """A non-zero return code of the C ABI, with the library's message."""

    def __init__(self, code: int, msg: str):
        super().__init__(f"[{code}] {msg}")
        self.code, self.msg = code, msg


def check(rc: int) -> None:
    if rc != 0:
        raise CbkvError(rc, load().cbkv_last_error().decode())
