"""The oracle against every known-answer test the reference holds for this path.

Each test restates one reference test (cited) with the same geometry, the same
deterministic input generators and the same assertions/tolerances, so the
oracle is pinned wherever the reference pins itself.
"""
import numpy as np
import pytest

import oracle
from oracle import OracleArena, OracleContiguous, OracleError


def paged(layers, max_seq_len, page_size, n_kv=2, d=8, dtype="f32", windows=None, rolling=True):
    a = OracleArena(layers, n_kv, d, max_seq_len, page_size, windows=windows, rolling=rolling, dtype=dtype)
    return a, a.new_seq()


# ---- kv.rs:1075-1114: allocator and config ---------------------------------
def test_allocator_alloc_in_order_and_exhaust():  # kv.rs:1075-1084
    a, s = paged(1, 3 * 16, 16)
    assert a.num_free_pages() == 3
    s.grow(48)
    assert list(s.block_table()) == [0, 1, 2]
    assert a.num_free_pages() == 0
    with pytest.raises(OracleError, match="page allocator exhausted"):
        s.grow(49)


def test_allocator_free_and_realloc_lifo():  # kv.rs:1086-1097
    a, s = paged(1, 32, 16)
    s.grow(32)
    p0, p1 = s.block_table()
    s.popn(32)  # table.pop() order frees p1 then p0
    assert a.num_free_pages() == 2
    s.grow(32)
    assert list(s.block_table()) == [p0, p1]


def test_allocator_reset_restores_all_pages():  # kv.rs:1099-1107
    a, s = paged(1, 64, 16)
    s.grow(32)
    s.reset()
    assert a.num_free_pages() == 4
    s.grow(1)
    assert list(s.block_table()) == [0]


@pytest.mark.parametrize("n,pages", [(16, 1), (17, 2), (1, 1)])
def test_cache_config_num_pages_rounds_up(n, pages):  # kv.rs:1109-1114
    a, _ = paged(1, n, 16)
    assert a.num_pages == pages and a.num_free_pages() == pages


# ---- kv.rs:1139-1192: page-table bookkeeping -------------------------------
def test_popn_frees_only_fully_unused_pages():  # kv.rs:1139-1160
    a, c = paged(2, 64, 16)
    c.grow(40)
    assert c.pages_used() == 3 and a.num_free_pages() == 1
    c.popn(9)
    assert c.seq_len() == 31 and c.pages_used() == 2 and a.num_free_pages() == 2
    c.popn(15)
    assert c.pages_used() == 1
    c.popn(1)
    assert c.pages_used() == 1
    c.popn(1000)
    assert c.seq_len() == 0 and c.pages_used() == 0 and a.num_free_pages() == 4


def test_popn_boundary_exact_page_edge():  # kv.rs:1162-1172
    a, c = paged(2, 64, 16)
    c.grow(32)
    c.popn(16)
    assert c.pages_used() == 1 and a.num_free_pages() == 3
    c.popn(16)
    assert c.pages_used() == 0 and a.num_free_pages() == 4


def test_regrowth_after_popn_reuses_freed_pages():  # kv.rs:1174-1182
    a, c = paged(2, 64, 16)
    c.grow(40)
    freed = c.block_table()[2]
    c.popn(9)
    c.grow(33)
    assert c.pages_used() == 3 and a.num_free_pages() == 1
    assert c.block_table()[2] == freed


def test_reset_releases_all_pages():  # kv.rs:1184-1192
    a, c = paged(2, 64, 16)
    c.grow(40)
    c.reset()
    assert c.seq_len() == 0 and c.pages_used() == 0 and a.num_free_pages() == 4


# ---- deterministic fixtures of the reference tests (kv.rs:863-882) ----------
def kv_tok(i, n_kv, d):
    def mk(salt):
        j = np.arange(n_kv * d)
        return (((i * 7 + j * 3 + salt) % 13).astype(np.float32) / 13.0 - 0.5).reshape(1, n_kv, 1, d)
    return mk(0), mk(5)


def q_tok(i, n_q, d):
    j = np.arange(n_q * d)
    return (((i * 11 + j * 5) % 17).astype(np.float32) / 17.0 - 0.5).reshape(1, n_q, 1, d)


def cat_toks(fn, rng_, n_h, d):
    return np.concatenate([fn(i, n_h, d) for i in rng_], axis=2)


# ---- kv.rs:996-1073: sliding layers ----------------------------------------
def test_sliding_layer_matches_masked_global():  # kv.rs:1001-1030
    n_kv, n_q, d, w = 2, 4, 4, 5
    scale = 1.0 / np.sqrt(d) * 0.9
    _, glob = paged(1, 64, 16, n_kv, d)
    _, slid = paged(1, 64, 16, n_kv, d, windows=[w])
    k7 = np.concatenate([kv_tok(i, n_kv, d)[0] for i in range(7)], axis=2)
    v7 = np.concatenate([kv_tok(i, n_kv, d)[1] for i in range(7)], axis=2)
    q7 = cat_toks(q_tok, range(7), n_q, d)
    a = glob.attention_opts(0, q7, k7, v7, 0, scale, w)
    b = slid.attention_opts(0, q7, k7, v7, 0, scale, w)
    assert np.abs(a - b).max() < 1e-5
    for i in range(7, 14):
        k, v = kv_tok(i, n_kv, d)
        q = q_tok(i, n_q, d)
        a = glob.attention_opts(0, q, k, v, i, scale, w)
        b = slid.attention_opts(0, q, k, v, i, scale, w)
        assert np.abs(a - b).max() < 1e-5, i
    assert slid.pages_used() == 0
    assert glob.pages_used() > 0
    assert slid.page_stats()["layers_sliding"] == 1 and slid.page_stats()["layers_materialized"] == 0


def test_sliding_popn_before_eviction_matches_replay():  # kv.rs:1034-1057
    n_kv, n_q, d, w = 2, 2, 4, 8
    _, cache = paged(1, 64, 16, n_kv, d, windows=[w])
    for i in range(4):
        k, v = kv_tok(i, n_kv, d)
        cache.attention_opts(0, q_tok(i, n_q, d), k, v, i, 0.4, w)
    assert cache.popn(2) == 2 and cache.seq_len() == 2
    _, fresh = paged(1, 64, 16, n_kv, d, windows=[w])
    for i in range(2):
        k, v = kv_tok(i, n_kv, d)
        fresh.attention_opts(0, q_tok(i, n_q, d), k, v, i, 0.4, w)
    k, v = kv_tok(9, n_kv, d)
    a = cache.attention_opts(0, q_tok(9, n_q, d), k, v, 2, 0.4, w)
    b = fresh.attention_opts(0, q_tok(9, n_q, d), k, v, 2, 0.4, w)
    assert np.abs(a - b).max() < 1e-5


def test_sliding_popn_after_eviction_refuses():  # kv.rs:1061-1073
    _, cache = paged(1, 64, 16, 1, 4, windows=[4])
    for i in range(6):
        k, v = kv_tok(i, 1, 4)
        cache.attention_opts(0, q_tok(i, 1, 4), k, v, i, 0.5, 4)
    assert cache.popn(1) == 0
    assert cache.seq_len() == 6
    assert cache.popn(0) == 0


def test_window_below_two_is_rejected():  # kv.rs:514-516
    with pytest.raises(OracleError, match="sliding window must be >= 2"):
        OracleArena(1, 1, 4, 64, windows=[1])


# ---- tests/kv_cache.rs ------------------------------------------------------
N_Q, N_KV, HEAD_DIM, SCALE = 4, 2, 8, 0.35


def rand_qkv(rng, seq):  # tests/kv_cache.rs:17-35 (seeded here; unseeded there)
    q = rng.normal(0.0, 1.0, (1, N_Q, seq, HEAD_DIM)).astype(np.float32)
    k = rng.normal(0.37, 0.8, (1, N_KV, seq, HEAD_DIM)).astype(np.float32)
    v = rng.normal(-0.11, 1.3, (1, N_KV, seq, HEAD_DIM)).astype(np.float32)
    return q, k, v


def test_paged_matches_contiguous_across_chunks_and_decodes():  # tests/kv_cache.rs:63-91
    rng = np.random.default_rng(1)
    contiguous = OracleContiguous(2, N_KV, HEAD_DIM)
    _, pg = paged(2, 64, 4, N_KV, HEAD_DIM)
    pos = 0
    for seq in [5, 7, 1, 1, 1]:
        q, k, v = rand_qkv(rng, seq)
        for layer in range(2):
            oc = contiguous.attention(layer, q, k, v, pos, SCALE)
            op = pg.attention(layer, q, k, v, pos, SCALE)
            assert np.abs(oc - op).max() < 1e-4
        pos += seq
        assert contiguous.seq_len() == pos and pg.seq_len() == pos
    assert pg.pages_used() == 4


def test_paged_popn_rollback_matches_fresh_history():  # tests/kv_cache.rs:95-126
    rng = np.random.default_rng(2)
    _, rolled = paged(2, 64, 4, N_KV, HEAD_DIM)
    fresh = OracleContiguous(2, N_KV, HEAD_DIM)
    q0, k0, v0 = rand_qkv(rng, 10)
    for layer in range(2):
        rolled.attention(layer, q0, k0, v0, 0, SCALE)
    rolled.popn(6)
    assert rolled.seq_len() == 4 and rolled.pages_used() == 1
    for layer in range(2):
        fresh.attention(layer, q0[:, :, :4], k0[:, :, :4], v0[:, :, :4], 0, SCALE)
    q1, k1, v1 = rand_qkv(rng, 3)
    for layer in range(2):
        a = rolled.attention(layer, q1, k1, v1, 4, SCALE)
        b = fresh.attention(layer, q1, k1, v1, 4, SCALE)
        assert np.abs(a - b).max() < 1e-4
    assert rolled.seq_len() == 7 and fresh.seq_len() == 7


def test_paged_unaligned_chunks_match_contiguous():  # tests/kv_cache.rs:130-146
    rng = np.random.default_rng(3)
    contiguous = OracleContiguous(1, N_KV, HEAD_DIM)
    _, pg = paged(1, 64, 4, N_KV, HEAD_DIM)
    pos = 0
    for seq in [3, 6, 5, 2]:
        q, k, v = rand_qkv(rng, seq)
        assert np.abs(contiguous.attention(0, q, k, v, pos, SCALE) - pg.attention(0, q, k, v, pos, SCALE)).max() < 1e-4
        pos += seq
    assert pg.seq_len() == 16 and pg.pages_used() == 4


def test_paged_reset_allows_fresh_reuse():  # tests/kv_cache.rs:149-164
    rng = np.random.default_rng(4)
    _, c = paged(1, 64, 4, N_KV, HEAD_DIM)
    c.attention(0, *rand_qkv(rng, 9), 0, SCALE)
    assert c.seq_len() == 9
    c.reset()
    assert c.seq_len() == 0 and c.pages_used() == 0
    ref = OracleContiguous(1, N_KV, HEAD_DIM)
    q, k, v = rand_qkv(rng, 5)
    assert np.abs(c.attention(0, q, k, v, 0, SCALE) - ref.attention(0, q, k, v, 0, SCALE)).max() < 1e-4


def test_paged_capacity_overflow_panics():  # tests/kv_cache.rs:167-173
    rng = np.random.default_rng(5)
    _, c = paged(1, 8, 4, N_KV, HEAD_DIM)
    with pytest.raises(OracleError, match="capacity exceeded"):
        c.attention(0, *rand_qkv(rng, 9), 0, SCALE)
    assert c.seq_len() == 0 and c.pages_used() == 0


def test_non_contiguous_append_is_rejected():  # kv.rs:671-674
    rng = np.random.default_rng(6)
    _, c = paged(1, 64, 4, N_KV, HEAD_DIM)
    with pytest.raises(OracleError, match="dense contiguous appends"):
        c.attention(0, *rand_qkv(rng, 2), 3, SCALE)


# ---- tests/attn_cliff.rs: xorshift64 inputs at SmolLM2 geometry -------------
def xorshift_data(n, seed):  # attn_cliff.rs:28-45
    x = np.uint64(seed | 1)
    out = np.empty(n, dtype=np.float32)
    m = (1 << 64) - 1
    x = int(x)
    for i in range(n):
        x ^= (x << 13) & m
        x ^= x >> 7
        x ^= (x << 17) & m
        out[i] = np.float32(np.float32((x >> 40) & 0xFFFFFFFF) / np.float32(1 << 24) * np.float32(2.0) - np.float32(1.0))
    return out


def attend_f64(q, k, v, pos, scale, window=None):
    """Independent float64 attention (not the oracle's code path)."""
    n_q, seq, d = q.shape[-3:]
    n_kv, total, _ = k.shape[-3:]
    q = q.reshape(n_q, seq, d).astype(np.float64)
    k = np.repeat(k.reshape(n_kv, total, d).astype(np.float64), n_q // n_kv, axis=0)
    v = np.repeat(v.reshape(n_kv, total, d).astype(np.float64), n_q // n_kv, axis=0)
    s = np.einsum("hqd,hkd->hqk", q, k) * scale
    qp = pos + np.arange(seq)[:, None]
    kp = np.arange(total)[None, :]
    bad = kp > qp
    if window is not None:
        bad |= kp + window - 1 < qp
    s = np.where(bad[None], -np.inf, s)
    s -= s.max(-1, keepdims=True)
    p = np.exp(s)
    p /= p.sum(-1, keepdims=True)
    return np.einsum("hqk,hkd->hqd", p, v).reshape(1, n_q, seq, d)


@pytest.mark.parametrize("s", [511, 512, 513, 600, 1024])
def test_kv_cache_attention_matches_cpu_above_cliff(s):  # attn_cliff.rs:498-544
    n_q, n_kv, d, scale = 9, 3, 64, 0.125
    q = xorshift_data(n_q * s * d, 11).reshape(1, n_q, s, d)
    k = xorshift_data(n_kv * s * d, 22).reshape(1, n_kv, s, d)
    v = xorshift_data(n_kv * s * d, 33).reshape(1, n_kv, s, d)
    ref = OracleContiguous(1, n_kv, d).attention(0, q, k, v, 0, scale)
    _, pg = paged(1, 2048, 16, n_kv, d)
    out = pg.attention(0, q, k, v, 0, scale)
    assert np.abs(out - ref).max() < 1e-3
    # and both against independent float64 math
    assert np.abs(out - attend_f64(q, k, v, 0, scale)).max() < 1e-5


def test_oracle_f16_build_matches_float64_within_storage_rounding():
    rng = np.random.default_rng(7)
    n_q, n_kv, d = 28, 4, 128
    a = OracleArena(1, n_kv, d, 4096, dtype="f16")
    s = a.new_seq()
    q = rng.standard_normal((1, n_q, 300, d)).astype(np.float16)
    k = rng.standard_normal((1, n_kv, 300, d)).astype(np.float16)
    v = rng.standard_normal((1, n_kv, 300, d)).astype(np.float16)
    out = s.attention(0, q, k, v, 0, 1 / np.sqrt(d))
    assert out.dtype == np.float16
    ref = attend_f64(q, k, v, 0, 1 / np.sqrt(d))
    # output is one f16 rounding away from exact math
    assert np.abs(out.astype(np.float64) - ref).max() < 2e-3
    q1 = rng.standard_normal((1, n_q, 1, d)).astype(np.float16)
    k1 = rng.standard_normal((1, n_kv, 1, d)).astype(np.float16)
    v1 = rng.standard_normal((1, n_kv, 1, d)).astype(np.float16)
    o1 = s.attention_opts(0, q1, k1, v1, 300, 0.07, 64)
    kk = np.concatenate([k, k1], axis=2)
    vv = np.concatenate([v, v1], axis=2)
    assert np.abs(o1.astype(np.float64) - attend_f64(q1, kk, vv, 300, 0.07, 64)).max() < 2e-3


# ---- kv.rs:893-990: int8 KV pages ------------------------------------------
def test_kv_quant_roundtrip_exact_on_grid_values():  # kv.rs:897-922
    d = 64
    data = np.array([(((i * 37) % 255) - 127) * 0.5 for i in range(2 * 3 * d)], dtype=np.float32)
    data[::32] = 63.5                      # absmax 63.5 per group => scale 0.5
    x = data.reshape(1, 2, 3, d)
    packed, scales = oracle.kv_quantize(x)
    assert packed.shape == (1, 2, 3, d // 4) and scales.shape == (1, 2, 3, d // 32)
    assert np.all(scales == 0.5)
    back = oracle.kv_dequantize(packed, scales, d)
    assert np.all(np.abs(back - x) < 1e-6)
    # the packing itself (kv.rs:276-283): lanes 0-2 offset binary, lane 3 signed
    q = np.round(x / 0.5).astype(np.int64).reshape(-1, 4)
    want = (q[:, 0] + 128) + (q[:, 1] + 128) * 256 + (q[:, 2] + 128) * 65536 + q[:, 3] * 16777216
    assert np.array_equal(packed.reshape(-1).astype(np.int64), want)
    assert want.max() <= 2 ** 31 - 1


def test_kv_quant_extreme_corner_is_i32_max():       # kv.rs:279-281
    x = np.full((1, 32), 127.0, dtype=np.float32)
    packed, scales = oracle.kv_quantize(x)
    assert scales[0, 0] == 1.0 and np.all(packed == 2 ** 31 - 1)
    x[0, 3::4] = -127.0
    packed, _ = oracle.kv_quantize(x)
    assert np.all(packed == 255 + 255 * 256 + 255 * 65536 - 127 * 16777216)
    assert np.array_equal(oracle.kv_dequantize(packed, np.ones((1, 1), np.float32), 32), x)


def test_kv_quant_error_bounded_by_half_step():      # kv.rs:926-953
    d = 64
    data = np.array([((i * 7919) % 1000) / 250.0 - 2.0 for i in range(2 * 5 * d)], dtype=np.float32)
    x = data.reshape(1, 2, 5, d)
    back = oracle.kv_dequantize(*oracle.kv_quantize(x), d).reshape(-1, 32)
    for g, chunk in enumerate(data.reshape(-1, 32)):
        assert np.all(np.abs(chunk - back[g]) <= np.abs(chunk).max() / 254.0 + 1e-6)


def test_quantized_paged_cache_matches_fp_within_tolerance():   # kv.rs:955-990
    n_kv, n_q, d = 2, 4, 32
    scale = 1.0 / np.sqrt(d) * 0.9
    _, fp = paged(1, 64, 16, n_kv, d)
    qa = OracleArena(1, n_kv, d, 64, 16, dtype="f32", quantize_kv=True)
    qn = qa.new_seq()
    k20, v20 = (np.concatenate([kv_tok(i, n_kv, d)[j] for i in range(20)], axis=2) for j in (0, 1))
    q20 = cat_toks(q_tok, range(20), n_q, d)
    a = fp.attention_opts(0, q20, k20, v20, 0, scale)
    b = qn.attention_opts(0, q20, k20, v20, 0, scale)
    assert np.all(np.abs(a - b) < 1e-2)
    for i in range(20, 30):
        k, v = kv_tok(i, n_kv, d)
        q = q_tok(i, n_q, d)
        a = fp.attention_opts(0, q, k, v, i, scale)
        b = qn.attention_opts(0, q, k, v, i, scale)
        assert np.all(np.abs(a - b) < 1e-2)
    assert qn.seq_len() == 30 and qn.pages_used() == 2      # page semantics unchanged, kv.rs:984-989
    assert qn.popn(14) == 14 and qn.pages_used() == 1
