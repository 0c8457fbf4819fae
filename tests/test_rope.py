"""Rotary embedding + QK norm fused into the append: the library's host tables against the
reference's known answers and the oracle (CPU), and the fused kernel against the oracle (GPU)."""
import math

import numpy as np
import pytest
import torch

import oracle
from combsengine_b200 import CbkvError, KVArena
from combsengine_b200 import rope as R
from oracle import OracleArena

from kvcase import assert_attention_close

SCALINGS = [
    None,
    dict(kind="linear", factor=2.0),
    dict(kind="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=8192),
    dict(kind="yarn", factor=4.0, original_max_position_embeddings=32768, beta_fast=32.0, beta_slow=1.0),
    dict(kind="yarn", factor=4.0, original_max_position_embeddings=32768, attention_factor=1.25),
    dict(kind="longrope", short_factor=[1.0 + 0.1 * i for i in range(32)], original_max_position_embeddings=4096, factor=32.0),
]


# ------------------------------------------------------------------ host (no GPU)
def test_library_frequencies_hold_the_reference_known_answers():
    # rope.rs:248-346
    inv, ms = R.scaled_inv_freq(8, 10000.0, R.RopeScaling(kind="linear", factor=2.0))
    assert np.all(np.abs(inv - [0.5, 0.05, 0.005, 0.0005]) < 1e-12) and ms == 1.0
    inv, ms = R.scaled_inv_freq(64, 500000.0, R.RopeScaling.from_dict(SCALINGS[2]))
    for i, e in [(0, 1.0), (8, 0.037606030931), (16, 0.000429556797), (24, 1.661967e-06), (31, 9.4183e-08)]:
        assert abs((inv[i] - e) / e) < 1e-6
    inv, ms = R.scaled_inv_freq(128, 1e6, R.RopeScaling.from_dict(SCALINGS[3]))
    for i, e in [(0, 1.0), (16, 0.03162277660168379), (32, 0.0006029411764705882), (48, 7.905694150420949e-06),
                 (63, 3.102344401879299e-07)]:
        assert abs((inv[i] - e) / e) < 1e-6
    assert abs(ms - 1.138629436112) < 1e-9
    inv, ms = R.scaled_inv_freq(8, 10000.0, R.RopeScaling(kind="longrope", short_factor=[1.0, 2.0, 4.0, 8.0],
                                                         original_max_position_embeddings=4096, factor=32.0))
    assert np.all(np.abs(inv - [1.0, 0.05, 0.0025, 0.000125]) < 1e-15) and abs(ms - math.sqrt(17.0 / 12.0)) < 1e-12


@pytest.mark.parametrize("sc", SCALINGS)
def test_library_tables_equal_the_oracle_tables(sc):
    cos, sin = R.build_tables_scaled(64, 500000.0, 300, R.RopeScaling.from_dict(sc))
    ocos, osin = oracle.rope_tables(64, 500000.0, 300, sc)
    assert np.array_equal(cos, ocos) and np.array_equal(sin, osin)
    assert np.array_equal(cos[:, :32], cos[:, 32:])          # half-split layout, rope.rs:139-148


def test_table_position_zero_is_identity_and_bad_configs_are_refused():
    cos, sin = R.build_tables(8, 10000.0, 4)                  # rope.rs:215-244
    assert np.all(np.abs(cos[0] - 1.0) < 1e-6) and np.all(np.abs(sin[0]) < 1e-6)
    for pos in range(4):
        for i, f in enumerate([1.0, 0.1, 0.01, 0.001]):
            assert abs(cos[pos, i] - math.cos(pos * f)) < 1e-5 and abs(sin[pos, i + 4] - math.sin(pos * f)) < 1e-5
    with pytest.raises(CbkvError, match="head_dim"):
        R.build_tables(6, 10000.0, 4)
    with pytest.raises(CbkvError, match="scaling"):
        R.build_tables_scaled(8, 10000.0, 4, R.RopeScaling(kind="ntk"))


# ------------------------------------------------------------------ GPU
def _rows(rng, heads, tokens, d, dtype=np.float16):
    return rng.standard_normal((heads, tokens, d)).astype(dtype)


def _oracle_prepare(q, k, pos, cos, sin, norm):
    """llama.rs:275-285 on one sequence's q [Hq,S,d], k [Hkv,S,d]."""
    if norm is not None:
        qw, kw, eps, gemma = norm
        if qw is not None:
            q = oracle.rms_norm(q, qw, eps, gemma)
        if kw is not None:
            k = oracle.rms_norm(k, kw, eps, gemma)
    return oracle.rope_apply(q, pos, cos, sin), oracle.rope_apply(k, pos, cos, sin)


def _run_case(n_q, n_kv, d, steps, theta=10000.0, scaling=None, norm=None, window=None, seed=0, n_seqs=2,
              pages_exact=True, max_len=256, quantize=False):
    rng = np.random.default_rng(seed)
    npages = n_seqs * ((max_len + 15) // 16)
    g = KVArena(1, n_q, n_kv, d, max_len, num_pages=npages, quantize_kv=quantize)
    o = OracleArena(1, n_kv, d, max_len, num_pages=npages, rolling=False, dtype="f16", quantize_kv=quantize)
    perm = rng.permutation(npages)
    g.set_free_list(perm); o.set_free_list(perm)
    gs = [g.new_seq() for _ in range(n_seqs)]
    os_ = [o.new_seq() for _ in range(n_seqs)]
    rope = R.RotaryEmbedding(g, theta, max_len, R.RopeScaling.from_dict(scaling))
    cos, sin = oracle.rope_tables(d, theta, max_len, scaling)
    gnorm = onorm = None
    if norm is not None:
        qw = (rng.standard_normal(d) * 0.2 + (0.0 if norm == "gemma" else 1.0)).astype(np.float16)
        kw = (rng.standard_normal(d) * 0.2 + (0.0 if norm == "gemma" else 1.0)).astype(np.float16)
        gnorm = R.QKNorm(torch.from_numpy(qw).cuda(), torch.from_numpy(kw).cuda(), 1e-6, norm == "gemma")
        onorm = (qw, kw, 1e-6, norm == "gemma")
    scale = d ** -0.5
    for step, new in enumerate(steps):
        new = list(new)[:n_seqs]
        pos = [s.seq_len() for s in gs]
        q = [_rows(rng, n_q, n, d) for n in new]
        k = [_rows(rng, n_kv, n, d) for n in new]
        v = [_rows(rng, n_kv, n, d) for n in new]
        cat = lambda xs: torch.from_numpy(np.concatenate([x.reshape(-1) for x in xs])).cuda()
        g.begin_step(gs, new)
        got = R.attention_rope(g, 0, rope, cat(q), cat(k), cat(v), scale, window, gnorm).cpu().numpy()
        o.batch_begin(os_, new)
        qr, kr = zip(*[_oracle_prepare(q[b], k[b], pos[b], cos, sin, onorm) for b in range(n_seqs)])
        flat = lambda xs: np.concatenate([x.reshape(-1) for x in xs])
        ref = o.batch_layer(os_, new, 0, flat(qr), flat(kr), flat(v), n_q, scale, window)
        assert_attention_close(got, ref, f"step {step}")
    assert g.device_status() == 0
    for b in range(n_seqs):
        assert list(gs[b].block_table()) == list(os_[b].block_table())
        for page in gs[b].block_table():
            if quantize:  # rotated k, then kv_quantize: packed words and scales bit for bit
                for x, y in zip(g.export_page_quant(0, int(page)), o.page_quant(0, int(page))):
                    assert np.array_equal(x, y if y.dtype == np.int32 else y.view(np.uint16))
                continue
            gk, gv = g.export_page(0, int(page))
            ok, ov = o.page(0, int(page))
            assert np.array_equal(gv, ov.view(np.uint16)), "V pages are a bit copy"
            if pages_exact:
                assert np.array_equal(gk, ok.view(np.uint16)), "rotated K pages are bit-exact"
            else:  # the norm's sum of squares has no defined order: one f16 ulp
                assert np.allclose(gk.view(np.float16).astype(np.float32), ok.astype(np.float32), rtol=2e-3, atol=2e-3)
    rope.close()


@pytest.mark.gpu
@pytest.mark.parametrize("n_q,n_kv,d", [(9, 3, 64), (28, 4, 128), (8, 4, 256), (6, 2, 96)])
def test_rotated_append_and_attention_match_the_oracle(n_q, n_kv, d):
    _run_case(n_q, n_kv, d, [(70, 33), (1, 1), (1, 1), (5, 1), (1, 1)], seed=d)


@pytest.mark.gpu
@pytest.mark.parametrize("sc", SCALINGS[1:4])
def test_scaled_tables_on_the_device(sc):
    _run_case(8, 2, 64, [(40, 40), (1, 1), (1, 1)], theta=500000.0, scaling=sc, seed=5)


@pytest.mark.gpu
@pytest.mark.parametrize("flavour", ["rms", "gemma"])
def test_qk_norm_before_the_rotation(flavour):
    _run_case(8, 4, 256, [(50, 20), (1, 1), (1, 1), (1, 1)], norm=flavour, window=32, seed=9, pages_exact=False)
    _run_case(16, 8, 128, [(64, 64), (1, 1)], norm=flavour, seed=10, pages_exact=False)


@pytest.mark.gpu
def test_rotate_and_append_alone_is_bit_exact_and_may_run_in_place():
    rng = np.random.default_rng(21)
    n_q, n_kv, d, L = 12, 4, 128, 200
    g = KVArena(1, n_q, n_kv, d, 256, num_pages=16)
    s = g.new_seq()
    rope = R.RotaryEmbedding(g, 1e6, 256)
    cos, sin = oracle.rope_tables(d, 1e6, 256)
    q, k, v = _rows(rng, n_q, L, d), _rows(rng, n_kv, L, d), _rows(rng, n_kv, L, d)
    g.begin_step([s], [L])
    qd = torch.from_numpy(q.reshape(-1)).cuda()
    out = R.rope_append(g, 0, rope, qd, torch.from_numpy(k.reshape(-1)).cuda(), torch.from_numpy(v.reshape(-1)).cuda(), q_out=qd)
    assert out.data_ptr() == qd.data_ptr()
    ref_q = oracle.rope_apply(q, 0, cos, sin)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), ref_q.reshape(-1).view(np.uint16))
    ref_k = oracle.rope_apply(k, 0, cos, sin)
    for lp, page in enumerate(s.block_table()):
        gk, gv = g.export_page(0, int(page))
        n = min(16, L - lp * 16)
        assert np.array_equal(gk[:, :n], ref_k[:, lp * 16:lp * 16 + n].view(np.uint16))
        assert np.array_equal(gv[:, :n], v[:, lp * 16:lp * 16 + n].view(np.uint16))
    # a step past the table is refused before anything is launched
    g.begin_step([s], [56])
    small = R.RotaryEmbedding(g, 1e6, 220)
    z = torch.zeros(56 * n_q * d, dtype=torch.float16, device="cuda")
    zk = torch.zeros(56 * n_kv * d, dtype=torch.float16, device="cuda")
    with pytest.raises(CbkvError, match="rope table shorter"):
        R.rope_append(g, 0, small, z, zk, zk)


@pytest.mark.gpu
@pytest.mark.parametrize("n_q,n_kv,d", [(28, 4, 128), (8, 4, 64)])
def test_rotation_into_int8_pages(n_q, n_kv, d):
    _run_case(n_q, n_kv, d, [(70, 33), (1, 1), (1, 1), (5, 1), (1, 1)], seed=3 * d, quantize=True)
