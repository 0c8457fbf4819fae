"""The Rust declarations under bindings/rust follow include/combs_kv.h (no Rust toolchain needed).

The crate cannot be compiled where this repository is built, so this is the check that keeps it
honest: every function the header declares has a ``pub fn`` in ``combs-kv-sys/src/lib.rs`` with
the same number of parameters and a return type of the same width, every struct has the same
fields in the same order, and nothing is declared in Rust that the header does not have.
"""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "combs_kv.h")
SYS = os.path.join(ROOT, "bindings", "rust", "combs-kv-sys", "src", "lib.rs")
IMPL = os.path.join(ROOT, "bindings", "rust", "kv_b200.rs")


def _strip_c_comments(text: str) -> str:
    return re.sub(r"/\*.*?\*/", " ", text, flags=re.S)


def header_functions() -> dict:
    text = _strip_c_comments(open(HEADER).read())
    out = {}
    for m in re.finditer(r"\b(const\s+char\s*\*|int32_t|int64_t)\s+(cbkv_\w+)\s*\(([^;{]*?)\)\s*;", text, flags=re.S):
        ret, name, params = m.group(1), m.group(2), " ".join(m.group(3).split())
        n = 0 if params in ("", "void") else len(params.split(","))
        out[name] = (re.sub(r"\s+", "", ret), n)
    return out


def rust_functions() -> dict:
    text = re.sub(r"//.*", "", open(SYS).read())
    out = {}
    for m in re.finditer(r"pub\s+fn\s+(cbkv_\w+)\s*\(([^)]*)\)\s*(?:->\s*([^;]+))?;", text, flags=re.S):
        name, params, ret = m.group(1), " ".join(m.group(2).split()), (m.group(3) or "").strip()
        n = 0 if not params else len([p for p in params.split(",") if p.strip()])
        out[name] = (ret, n)
    return out


RET = {"int32_t": "i32", "int64_t": "i64", "constchar*": "*const c_char"}


def test_every_header_function_has_a_rust_declaration_and_nothing_else():
    h, r = header_functions(), rust_functions()
    assert len(h) >= 55, "the header parser lost declarations"
    assert sorted(set(h) - set(r)) == [], "declared in combs_kv.h but missing in combs-kv-sys"
    assert sorted(set(r) - set(h)) == [], "declared in combs-kv-sys but not in combs_kv.h"
    for name, (ret, n) in h.items():
        rret, rn = r[name]
        assert rn == n, f"{name}: {n} parameters in C, {rn} in Rust"
        assert rret == RET[ret], f"{name}: returns {ret} in C, {rret} in Rust"


def _c_struct_fields(name: str) -> list:
    text = _strip_c_comments(open(HEADER).read())
    m = re.search(r"typedef\s+struct\s*(?:\w+\s*)?\{([^}]*)\}\s*" + name + r"\s*;", text, flags=re.S)
    assert m, name
    fields = []
    for decl in m.group(1).split(";"):
        if decl.strip():  # "double beta_fast, beta_slow" declares two
            fields += [re.search(r"(\w+)\s*$", part.strip()).group(1) for part in decl.split(",")]
    return fields


def _rust_struct_fields(name: str) -> list:
    text = re.sub(r"//.*", "", open(SYS).read())
    m = re.search(r"pub\s+struct\s+" + name + r"\s*\{([^}]*)\}", text, flags=re.S)
    assert m, name
    return re.findall(r"pub\s+(\w+)\s*:", m.group(1))


def test_structs_have_the_same_fields_in_the_same_order():
    for name in ("cbkv_config", "cbkv_page_stats_t", "cbkv_rope_config", "cbkv_qk_norm"):
        assert _c_struct_fields(name) == _rust_struct_fields(name), name


def test_error_codes_agree():
    text = _strip_c_comments(open(HEADER).read())
    rust = open(SYS).read()
    codes = dict(re.findall(r"(CBKV_(?:OK|ERR_\w+))\s*=\s*(-?\d+)", text))
    assert len(codes) == 9
    for k, v in codes.items():
        assert re.search(r"pub const " + k + r": i32 = " + v + r";", rust), k


def test_the_trait_implementation_only_calls_declared_functions():
    used = set(re.findall(r"\b(cbkv_\w+)\s*\(", open(IMPL).read()))
    assert used and used <= set(rust_functions())
    src = open(IMPL).read()
    for method in ("attention_opts", "seq_len", "popn", "reset", "pages_used", "page_stats"):  # kv.rs:92-151
        assert re.search(r"fn\s+" + method + r"\b", src), method
