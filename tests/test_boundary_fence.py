"""No C++ exception and no null handle may take the host process down (CPU only).

The reference's C ABI wraps every entry point in ``catch_unwind`` and reports a panic as a return
code plus a thread-local message (combs-ffi/src/lib.rs:41-71,143,173-183); this library does the
same with C++ exceptions.  The dynamic part throws inside an entry point on purpose; the static
part reads the sources and fails when an ``extern "C"`` definition does not go through the fence.
"""
import ctypes as C
import os
import re

import pytest

from combsengine_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "combsengine_b200", "csrc")


@pytest.mark.parametrize("kind,text", [(1, b"out of host memory"), (2, b"raised on request"), (3, b"unknown C++ exception")])
def test_an_exception_inside_an_entry_point_becomes_a_return_code(kind, text):
    lib = _lib.load()
    assert lib.cbkv_debug_raise(kind) == -8  # CBKV_ERR_INTERNAL
    assert text in lib.cbkv_last_error()
    assert lib.cbkv_debug_raise(0) == 0      # and the library is still usable


def test_null_handles_are_errors_not_crashes():
    lib = _lib.load()
    assert lib.cbkv_seq_len(None) == -4
    assert lib.cbkv_pages_used(None) == -4
    assert lib.cbkv_num_free_pages(None) == -4
    assert lib.cbkv_page_bytes(None) == -4
    assert lib.cbkv_export_block_table(None, None, 0) == -4
    assert lib.cbkv_export_free_list(None, None, 0) == -4
    assert lib.cbkv_page_refcount(None, 0) == -4
    assert lib.cbkv_popn(None, 1, C.byref(C.c_int64(0))) == -4
    assert lib.cbkv_reset(None) == -4
    assert lib.cbkv_page_stats(None, None) == -4
    assert lib.cbkv_layer_is_quantized(None, 0) == -4
    assert lib.cbkv_sessions_count(None) == 0 and lib.cbkv_sessions_evictions(None) == 0  # no table: nothing in it
    assert lib.cbkv_sessions_history_len(None, b"x") == -1
    assert lib.cbkv_device_status(None, None, None) == -4
    assert lib.cbkv_static_status(None, None) == -4
    assert lib.cbkv_begin_step(None, None, None, None, 0, None) == -4
    assert lib.cbkv_seq_destroy(None) == 0 and lib.cbkv_arena_destroy(None) == 0  # destroying nothing is fine


def _definitions(path):
    """(name, body) of every cbkv_* function defined at file scope."""
    text = open(path).read()
    text = re.sub(r"//[^\n]*", "", text)
    out = []
    for m in re.finditer(r'^(?:extern "C" )?(?:int32_t|int64_t) (cbkv_\w+)\([^;{]*\)\s*\{', text, flags=re.M):
        depth, i = 0, m.end() - 1
        while True:
            depth += {"{": 1, "}": -1}.get(text[i], 0)
            if depth == 0:
                break
            i += 1
        out.append((m.group(1), text[m.end():i]))
    return out


def test_every_entry_point_runs_behind_the_fence():
    names = set()
    for f in ("api.cu", "sessions.cpp", "noalloc.cu"):
        for name, body in _definitions(os.path.join(CSRC, f)):
            names.add(name)
            assert re.match(r"\s*return fenced(64)?\(\[&\]\(\) -> int(32|64)_t \{", body), f"{name} in {f} is not fenced"
    declared = {n for n in _lib.PROTOTYPES if n != "cbkv_last_error"}
    assert declared <= names, sorted(declared - names)
