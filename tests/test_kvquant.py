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


@pytest.mark.gpu
def test_quantized_decode_streams_many_pages_and_reuses_the_ring():
    # long contexts, ragged lengths, a window: every CTA wraps its ring many times and segments are cut
    # across CTAs; decode runs on the record-streaming kernel, the fill on the generic one
    from oracle import OracleArena
    n_q, n_kv, d = 28, 4, 128
    rng = np.random.default_rng(31)
    lens = [3000, 1500, 777, 16, 1]
    pages = sum((L + 40) // 16 + 1 for L in lens)
    g = KVArena(1, n_q, n_kv, d, 3100, num_pages=pages, quantize_kv=True)
    o = OracleArena(1, n_kv, d, 3100, num_pages=pages, rolling=False, dtype="f16", quantize_kv=True)
    perm = rng.permutation(pages)
    g.set_free_list(perm); o.set_free_list(perm)
    gs, os_ = [g.new_seq() for _ in lens], [o.new_seq() for _ in lens]
    k = [rng.standard_normal((n_kv, L, d)).astype(np.float16) for L in lens]
    v = [rng.standard_normal((n_kv, L, d)).astype(np.float16) for L in lens]
    cat = lambda xs: torch.from_numpy(np.concatenate([x.reshape(-1) for x in xs])).cuda()
    g.begin_step(gs, lens)
    g.append(0, cat(k), cat(v))
    o.batch_begin(os_, lens)
    for b, s in enumerate(os_):
        s.append_only(0, k[b], v[b], 0)
    for step, window in enumerate([None, None, 1000, None]):
        one = [1] * len(lens)
        q, k1, v1 = ([rng.standard_normal((h, 1, d)).astype(np.float16) for _ in lens] for h in (n_q, n_kv, n_kv))
        g.begin_step(gs, one)
        got = g.attention(0, cat(q), cat(k1), cat(v1), d ** -0.5, window).cpu().numpy()
        o.batch_begin(os_, one)
        flat = lambda xs: np.concatenate([x.reshape(-1) for x in xs])
        ref = o.batch_layer(os_, one, 0, flat(q), flat(k1), flat(v1), n_q, d ** -0.5, window)
        from kvcase import assert_attention_close
        assert_attention_close(got, ref, f"decode step {step}")
    assert g.device_status() == 0
    for b in (0, 4):
        for pg in gs[b].block_table()[-2:]:
            for x, y in zip(g.export_page_quant(0, int(pg)), o.page_quant(0, int(pg))):
                assert np.array_equal(x, y if y.dtype == np.int32 else y.view(np.uint16))


@pytest.mark.gpu
def test_bf16_quantized_decode_against_a_float32_reading_of_its_own_pages():
    n_q, n_kv, d, L = 8, 2, 128, 333
    rng = np.random.default_rng(8)
    g = KVArena(1, n_q, n_kv, d, 512, quantize_kv=True, dtype=torch.bfloat16)
    s = g.new_seq()
    t = lambda x: torch.from_numpy(x).cuda().to(torch.bfloat16)
    k, v = rng.standard_normal((n_kv, L, d)).astype(np.float32), rng.standard_normal((n_kv, L, d)).astype(np.float32)
    g.begin_step([s], [L])
    g.append(0, t(k.reshape(-1)), t(v.reshape(-1)))
    q, k1, v1 = (rng.standard_normal((h, 1, d)).astype(np.float32) for h in (n_q, n_kv, n_kv))
    g.begin_step([s], [1])
    got = g.attention(0, t(q.reshape(-1)), t(k1.reshape(-1)), t(v1.reshape(-1)), d ** -0.5).float().cpu().numpy().reshape(n_q, d)
    # read the pages back and de-quantise them by the reference's rule (kv.rs:319-358) in float32
    K, V = np.zeros((n_kv, L + 1, d), np.float32), np.zeros((n_kv, L + 1, d), np.float32)
    for lp, pg in enumerate(s.block_table()):
        kp, ks, vp, vs = g.export_page_quant(0, int(pg))
        n = min(16, L + 1 - lp * 16)
        for packed, scales, dst in ((kp, ks, K), (vp, vs, V)):
            by = packed.view(np.uint8).reshape(n_kv, 16, d).astype(np.int32)
            qv = np.where(np.arange(d) % 4 == 3, by.astype(np.int8).astype(np.int32), by - 128)
            sc = torch.from_numpy(scales.astype(np.int16)).view(torch.bfloat16).float().numpy()      # [n_kv, 16, d/32]
            dq = torch.from_numpy(qv.astype(np.float32) * np.repeat(sc, 32, axis=-1)).to(torch.bfloat16).float().numpy()
            dst[:, lp * 16:lp * 16 + n] = dq[:, :n]
    qb = torch.from_numpy(q).to(torch.bfloat16).float().numpy().reshape(n_q, d)
    ref = np.zeros((n_q, d), np.float32)
    for h in range(n_q):
        sc = (K[h // (n_q // n_kv)] @ qb[h]) * d ** -0.5
        p = np.exp(sc - sc.max()); p /= p.sum()
        ref[h] = p @ V[h // (n_q // n_kv)]
    assert np.abs(got - ref).max() < 2e-2, np.abs(got - ref).max()


@pytest.mark.gpu
@pytest.mark.parametrize("n_q,n_kv,d,chunks", [(32, 8, 128, (300, 150)), (9, 3, 64, (200, 90)), (8, 4, 256, (130, 40))])
def test_chunks_over_int8_layers_run_on_the_tensor_core_kernels(n_q, n_kv, d, chunks):
    # chunk steps de-quantise the sequences' pages into a float scratch layer and run the chunk kernels over it
    p = Pair(2, n_q, n_kv, d, 1024, num_pages=120, seed=7 + d, shuffle_free_list=True, quantize_kv=True)
    a, b = p.new_seq(), p.new_seq()
    p.step([a, b], list(chunks))
    p.step([a, b], [1, 1])
    p.step([a, b], [chunks[1], chunks[0]], window=200)     # a second chunk over the cached prefix, with a window
    p.step([a, b], [1, 1])
    p.assert_state_equal(pages="used")


@pytest.mark.gpu
@pytest.mark.parametrize("n_q", [32, 28])
def test_two_tile_kernel_converts_int8_records_itself(n_q):
    # chunk kernel mode 4: no float copy, the tcgen05 kernel fetches the half-records of every page and
    # converts them in registers; same tolerance against the oracle as the default route, and the same
    # result as that route to within float rounding of the output
    outs = []
    for mode in (4, 0):
        p = Pair(2, n_q, 4, 128, 4096, num_pages=400, seed=41, shuffle_free_list=True, quantize_kv=True, chunk_kernel=mode)
        a, b, c = p.new_seq(), p.new_seq(), p.new_seq()
        p.step([a, b, c], [700, 130, 257])                  # several K/V tiles per CTA, ragged last pages
        p.step([a, b], [1, 1])
        outs.append(p.step([a, c], [256, 300], window=500))  # a second chunk over the cached prefix, with a window
        p.step([a, b, c], [1, 1, 1])
        p.assert_state_equal(pages="used")
    if outs[0] is not None:
        np.testing.assert_allclose(np.asarray(outs[0], np.float32), np.asarray(outs[1], np.float32), atol=2e-3, rtol=1e-2)


@pytest.mark.gpu
def test_int8_pages_with_prefix_sharing_and_churn():
    # shared prefix pages (refcounted), decode with the quantising append inside the kernel, rollback to the
    # prefix and replacement: private pages only are ever written, packed records stay bit-exact
    p = Pair(2, 28, 4, 128, 2048, num_pages=300, shuffle_free_list=True, seed=0xC0B5, popn_refuses=False, quantize_kv=True)
    root = p.new_seq()
    p.step([root], [64])
    live = [p.fork(root, 64) for _ in range(8)]
    p.step(live, [int(x) for x in p.rng.integers(8, 200, len(live))], check=False)
    for it in range(2):
        for _ in range(4):
            p.step(live, [1] * len(live))
        e = live[int(p.rng.integers(len(live)))]
        n = e[0].seq_len() - 64
        assert e[0].popn(n) == n and e[1].popn(n) == n
        live.remove(e)
        p.drop(e)
        live.append(p.fork(root, 64))
        p.step(live[-1:], [int(p.rng.integers(20, 90))], check=False)
    p.step(live, [1] * len(live))
    p.assert_state_equal(pages="used")
