"""int8 KV pages (CacheConfig::quantize_kv, kv.rs:271-358,464-475,740-787): packed words and scales
bit-exact against the oracle, attention within the path's tolerance, page semantics unchanged."""
import numpy as np
import pytest
import torch

import oracle
from combsengine_b200 import CbkvError, KVArena
from kvcase import Pair


# ------------------------------------------------------------------ host (no GPU)
def test_which_layers_are_quantized_and_what_a_page_costs():
    a = KVArena(3, 8, 2, 64, 128, num_pages=8, windows=[None, 16, None], quantize_kv=True)
    assert [a.layer_is_quantized(l) for l in range(3)] == [True, False, True]   # kv.rs:688-694
    rec = 2 * 16 * 64 + 2 * 16 * 2 * 2                 # bytes + scales of K and V, one head
    assert a.page_bytes() == 2 * (2 * rec) + 16 * 2 * 64 * 2 * 2
    b = KVArena(1, 8, 2, 40, 128, num_pages=8, quantize_kv=True)          # head_dim % 32 != 0: float pages
    assert not b.layer_is_quantized(0)
    c = KVArena(1, 8, 2, 64, 128, num_pages=8)
    assert not c.layer_is_quantized(0)
    kp, ks, vp, vs = a.export_page_quant(0, 3)                           # never written: zeros
    assert not kp.any() and not ks.any() and not vp.any() and not vs.any()
    with pytest.raises(CbkvError, match="float pages"):
        a.export_page_quant(1, 0)


# ------------------------------------------------------------------ GPU
@pytest.mark.gpu
@pytest.mark.parametrize("n_q,n_kv,d", [(28, 4, 128), (9, 3, 64), (8, 4, 256), (6, 2, 96)])
def test_quantized_pages_and_attention_match_the_oracle(n_q, n_kv, d):
    p = Pair(2, n_q, n_kv, d, 256, num_pages=40, seed=d, shuffle_free_list=True, quantize_kv=True)
    a, b = p.new_seq(), p.new_seq()
    p.step([a, b], [37, 70])
    for _ in range(4):
        p.step([a, b], [1, 1])
    p.step([a, b], [5, 1])
    assert a[0].popn(9) == a[1].popn(9) == 9
    p.step([a, b], [1, 1], window=24)
    p.step([a], [20])
    p.assert_state_equal()


@pytest.mark.gpu
def test_window_layers_keep_float_pages_next_to_quantized_ones():
    p = Pair(3, 8, 4, 128, 200, num_pages=30, windows=[None, 32, None], seed=4, quantize_kv=True, popn_refuses=False)
    a = p.new_seq()
    p.step([a], [90])
    for _ in range(6):
        p.step([a], [1])
    assert [p.g.layer_is_quantized(l) for l in range(3)] == [True, False, True]
    p.assert_state_equal(pages="used")


@pytest.mark.gpu
def test_reference_grid_values_pack_exactly_on_the_device():
    # kv.rs:897-922: values that are exact multiples of the group scale survive bit for bit
    d, n_kv, T = 64, 2, 3
    data = np.array([(((i * 37) % 255) - 127) * 0.5 for i in range(n_kv * T * d)], dtype=np.float32)
    data[::32] = 63.5
    x = data.reshape(n_kv, T, d).astype(np.float16)
    g = KVArena(1, 4, n_kv, d, 64, num_pages=4, quantize_kv=True)
    s = g.new_seq()
    g.begin_step([s], [T])
    g.append(0, torch.from_numpy(x.reshape(-1)).cuda(), torch.from_numpy(x.reshape(-1)).cuda())
    kp, ks, vp, vs = g.export_page_quant(0, int(s.block_table()[0]))
    want_p, want_s = oracle.kv_quantize(x)
    assert np.array_equal(kp[:, :T], want_p) and np.array_equal(vp[:, :T], want_p)
    assert np.array_equal(ks[:, :T], want_s.view(np.uint16)) and np.all(want_s == 0.5)
    back = oracle.kv_dequantize(kp[:, :T], ks[:, :T].view(np.float16), d)
    assert np.array_equal(back, x)


@pytest.mark.gpu
def test_quantized_cache_tracks_the_float_cache():
    # kv.rs:955-990 / :1250-1272 (production backend tolerance 5e-2), on the reference's closed-form fixtures
    n_kv, n_q, d = 2, 4, 32
    scale = 1.0 / np.sqrt(d) * 0.9

    def kv_tok(i, salt):
        j = np.arange(n_kv * d)
        return (((i * 7 + j * 3 + salt) % 13).astype(np.float32) / 13.0 - 0.5).reshape(n_kv, 1, d).astype(np.float16)

    def q_tok(i):
        j = np.arange(n_q * d)
        return (((i * 11 + j * 5) % 17).astype(np.float32) / 17.0 - 0.5).reshape(n_q, 1, d).astype(np.float16)

    fp = KVArena(1, n_q, n_kv, d, 64)
    qn = KVArena(1, n_q, n_kv, d, 64, quantize_kv=True)
    sf, sq = fp.new_seq(), qn.new_seq()
    dev = lambda x: torch.from_numpy(np.ascontiguousarray(x).reshape(-1)).cuda()
    k20 = np.concatenate([kv_tok(i, 0) for i in range(20)], axis=1)
    v20 = np.concatenate([kv_tok(i, 5) for i in range(20)], axis=1)
    q20 = np.concatenate([q_tok(i) for i in range(20)], axis=1)
    outs = []
    for arena, s in ((fp, sf), (qn, sq)):
        arena.begin_step([s], [20])
        outs.append(arena.attention(0, dev(q20), dev(k20), dev(v20), scale).float().cpu().numpy())
    assert np.all(np.abs(outs[0] - outs[1]) < 5e-2)
    for i in range(20, 30):
        outs = []
        for arena, s in ((fp, sf), (qn, sq)):
            arena.begin_step([s], [1], [i])
            outs.append(arena.attention(0, dev(q_tok(i)), dev(kv_tok(i, 0)), dev(kv_tok(i, 5)), scale).float().cpu().numpy())
        assert np.all(np.isfinite(outs[1])) and np.all(np.abs(outs[0] - outs[1]) < 5e-2)
    assert sq.seq_len() == 30 and sq.pages_used() == 2
