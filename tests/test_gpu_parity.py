"""CUDA path vs oracle on identical seeded inputs, through the C ABI (needs a B200).

Small versions of the five benchmark configurations plus the reference's own test
patterns; page contents, block tables and free-list are compared bit for bit,
attention outputs within |err| <= 2e-3 + 1e-2 |ref| (f16 storage, f32 accumulation).
"""
import numpy as np
import pytest
import torch

from kvcase import Pair, assert_attention_close

pytestmark = pytest.mark.gpu


def test_cfg1_smollm2_prefill_decode_popn_reappend():
    # 9 q heads, 3 kv heads, d 64, one layer, 64 pages in a seeded shuffle
    p = Pair(1, 9, 3, 64, 1024, shuffle_free_list=True, seed=0xC0B50001)
    s = p.new_seq()
    p.step([s], [512])
    assert s[0].pages_used() == 32
    for _ in range(128):
        p.step([s], [1])
    assert s[0].seq_len() == 640
    p.assert_state_equal()
    assert s[0].popn(32) == 32 and s[1].popn(32) == 32
    p.assert_state_equal()
    for _ in range(32):
        p.step([s], [1])
    p.assert_state_equal()  # stale rows of popped tokens were overwritten identically


@pytest.mark.parametrize("fused", [True, False])
def test_cfg2_qwen_batched_decode_scattered_pages(fused):
    p = Pair(2, 28, 4, 128, 4096, num_pages=512, shuffle_free_list=True, seed=0xC0B50002)
    seqs = [p.new_seq() for _ in range(8)]
    lens = [int(x) for x in p.rng.integers(60, 700, len(seqs))]
    lens[0], lens[1] = 15, 16  # page edges
    p.step(seqs, lens, check=False)
    for _ in range(20):
        p.step(seqs, [1] * len(seqs), fused=fused)
    p.assert_state_equal(pages="used")


@pytest.mark.parametrize("consumers,stages,overlap", [(4, 4, True), (4, 8, False), (6, 6, True), (8, 8, True), (8, 16, False)])
def test_decode_ring_is_reused_many_times(consumers, stages, overlap):
    # few CTAs and a short TMA ring: every stage is refilled dozens of times per launch
    p = Pair(2, 28, 4, 128, 2048, num_pages=700, shuffle_free_list=True, seed=consumers * 100 + stages,
             tuning=dict(stages=stages, consumers=consumers, max_ctas=3, overlap_launches=overlap))
    seqs = [p.new_seq() for _ in range(6)]
    p.step(seqs, [int(x) for x in p.rng.integers(500, 1500, len(seqs))], check=False)
    for _ in range(4):
        p.step(seqs, [1] * len(seqs))
    p.assert_state_equal(pages="used")


def test_cfg3_gemma_windows_over_paged_kv():
    # 5 local : 1 global, d 256; window shortened so that it slides within the test
    windows = [96, 96, None, 96]
    p = Pair(4, 8, 4, 256, 2048, num_pages=256, windows=windows, seed=0xC0B50003)
    seqs = [p.new_seq() for _ in range(4)]
    p.step(seqs, [40, 95, 96, 300])
    for _ in range(40):
        p.step(seqs, [1, 1, 1, 1])
    p.assert_state_equal(pages="used")
    assert seqs[3][0].popn(1) == 0  # a sliding layer would have evicted: refused, kv.rs:812-816
    assert seqs[3][0].seq_len() == 340
    assert seqs[0][0].popn(1) == 1  # 80 tokens <= w - 1: nothing evicted yet


def test_cfg3_explicit_window_argument_on_global_layers():  # kv.rs:1001-1030, the masked-global side
    p = Pair(1, 8, 4, 256, 1024, seed=5)
    s = p.new_seq()
    p.step([s], [7], scale=0.9 / 16, window=5)
    for _ in range(30):
        p.step([s], [1], scale=0.9 / 16, window=5)


@pytest.mark.parametrize("chunk_kernel", [1, 2, 3])
def test_cfg4_llama_chunked_prefill(chunk_kernel):
    p = Pair(2, 32, 8, 128, 2048, num_pages=256, shuffle_free_list=True, seed=0xC0B50004, chunk_kernel=chunk_kernel)
    seqs = [p.new_seq(), p.new_seq()]
    for _ in range(3):
        p.step(seqs, [128, 128])
    p.step(seqs, [100, 37])      # ragged, not page aligned
    p.step(seqs, [1, 64])        # a decode row next to a chunk
    p.assert_state_equal(pages="used")


@pytest.mark.parametrize("geom", [(28, 4, 128, 2), (9, 3, 64, 2), (8, 8, 128, 2), (16, 2, 64, 2),
                                  (8, 4, 256, 2), (16, 2, 256, 2), (4, 4, 256, 2),
                                  (28, 4, 128, 3), (8, 8, 128, 3), (16, 2, 128, 3)])
def test_tensor_core_chunk_kernel_shapes_windows_and_ragged_chunks(geom):
    # tcgen05 kernels forced: q-head groups of 7, 3, 1 and 8; windows; chunks that do not fill a tile
    n_q, n_kv, d, kernel = geom
    p = Pair(2, n_q, n_kv, d, 4096, num_pages=300, shuffle_free_list=True, seed=n_q * 7 + d, windows=[None, 200],
             chunk_kernel=kernel, popn_refuses=False)
    seqs = [p.new_seq(), p.new_seq(), p.new_seq()]
    p.step(seqs, [300, 17, 129])
    p.step(seqs, [130, 256, 1])
    p.step(seqs, [5, 40, 64], scale=0.05)
    p.assert_state_equal(pages="used")


def test_cfg5_prefix_sharing_and_churn():
    p = Pair(2, 28, 4, 128, 4096, num_pages=400, shuffle_free_list=True, seed=0xC0B50005, popn_refuses=False)
    root = p.new_seq()
    p.step([root], [64])
    live = [p.fork(root, 64) for _ in range(12)]
    suffix = np.round(np.exp(p.rng.uniform(np.log(8), np.log(300), len(live)))).astype(int)
    p.step(live, [int(x) for x in suffix], check=False)
    for it in range(3):
        for _ in range(6):
            p.step(live, [1] * len(live))
        evict = [live[i] for i in p.rng.permutation(len(live))[:2]]
        for e in evict:  # back to the shared prefix; private pages return to the LIFO free-list
            n = e[0].seq_len() - 64
            assert e[0].popn(n) == n and e[1].popn(n) == n
        p.assert_state_equal(pages="used")
        for e in evict:
            live.remove(e)
            p.drop(e)
            live.append(p.fork(root, 64))
        p.step(live[-2:], [int(x) for x in p.rng.integers(20, 90, 2)], check=False)
    p.step(live, [1] * len(live))
    p.assert_state_equal(pages="used")


@pytest.mark.parametrize("chunks", [[5, 7, 1, 1, 1], [3, 6, 5, 2]])
def test_reference_chunk_patterns_at_reference_geometry(chunks):
    # tests/kv_cache.rs:63-146: page size 4, 4 q / 2 kv heads, d 8 -> the generic kernel
    p = Pair(2, 4, 2, 8, 64, page_size=4, seed=7)
    s = p.new_seq()
    for n in chunks:
        p.step([s], [n], scale=0.35)
    assert s[0].pages_used() == 4
    p.assert_state_equal()


def test_reference_popn_rollback_then_new_tokens():  # tests/kv_cache.rs:95-126
    p = Pair(2, 4, 2, 64, 64, seed=8)
    s = p.new_seq()
    p.step([s], [40], scale=0.35)
    assert s[0].popn(24) == 24 and s[1].popn(24) == 24
    assert s[0].pages_used() == 1
    p.step([s], [3], scale=0.35)
    assert s[0].seq_len() == 19
    p.assert_state_equal()
    s[0].reset(); s[1].reset()   # tests/kv_cache.rs:149-164
    p.step([s], [5], scale=0.35)
    p.assert_state_equal()


def test_bf16_storage_runs_and_tracks_f32_math():
    from combsengine_b200 import KVArena
    torch.manual_seed(0)
    a = KVArena(1, 8, 2, 128, 512, dtype=torch.bfloat16)
    s = a.new_seq()
    a.begin_step([s], [200])
    q = torch.randn(8, 200, 128, device="cuda").bfloat16()
    k = torch.randn(2, 200, 128, device="cuda").bfloat16()
    v = torch.randn(2, 200, 128, device="cuda").bfloat16()
    out = a.attention(0, q, k, v, 128 ** -0.5).float()
    kk, vv = k.float().repeat_interleave(4, 0), v.float().repeat_interleave(4, 0)
    sc = torch.einsum("hqd,hkd->hqk", q.float(), kk) * 128 ** -0.5
    sc = sc.masked_fill(torch.ones(200, 200, device="cuda").triu(1).bool(), float("-inf"))
    ref = torch.einsum("hqk,hkd->hqd", sc.softmax(-1), vv)
    assert (out - ref).abs().max().item() < 3e-2  # bf16 probabilities and output
    assert a.device_status() == 0


def test_host_buffer_entry_point_matches_device_one():
    p = Pair(1, 28, 4, 128, 1024, seed=11)
    s = p.new_seq()
    p.step([s], [300], check=False)
    g = p.g
    g.begin_step([s[0]], [1])
    q = torch.randn(28 * 128).half().pin_memory()
    k = torch.randn(4 * 128).half().pin_memory()
    v = torch.randn(4 * 128).half().pin_memory()
    out = torch.empty_like(q).pin_memory()
    g.attention_host(0, q, k, v, out, 0.1)
    s[0].popn(1)
    g.begin_step([s[0]], [1])
    ref = g.attention(0, q.cuda(), k.cuda(), v.cuda(), 0.1).cpu()
    assert torch.equal(out, ref)
    # pipelined variant: six calls in flight over four staging slots, outputs valid after host_sync
    outs = [torch.empty_like(q).pin_memory() for _ in range(6)]
    qs = [torch.randn(28 * 128).half().pin_memory() for _ in range(6)]
    refs = []
    for i in range(6):
        s[0].popn(1)
        g.begin_step([s[0]], [1])
        g.attention_host_async(0, qs[i], k, v, outs[i], 0.1)
    g.host_sync()
    for i in range(6):
        s[0].popn(1)
        g.begin_step([s[0]], [1])
        refs.append(g.attention(0, qs[i].cuda(), k.cuda(), v.cuda(), 0.1).cpu())
    for o, r in zip(outs, refs):
        assert torch.equal(o, r)


@pytest.mark.parametrize("direct", [True, False])
def test_host_buffer_pipeline_over_many_layers_and_steps(direct):
    # Decode steps over 5 layers through attention_host_async, 9 steps without a host_sync in between: 45 calls
    # over the 32 rotating slots, the kernels waiting for their inputs' flag (direct) or the stream waiting for
    # the input copies' event; pinned and pageable outputs mixed.  Every output must equal the device entry
    # point's.
    layers, n_q, n_kv, d = 5, 28, 4, 128
    p = Pair(layers, n_q, n_kv, d, 2048, num_pages=400, seed=23, shuffle_free_list=True)
    seqs = [p.new_seq() for _ in range(3)]
    p.step(seqs, [300, 17, 130], check=False)
    g = p.g
    g.set_host_route(direct)
    gs = [s[0] for s in seqs]
    n = len(gs)
    steps = 9
    mk = lambda heads, pinned: (torch.randn(n * heads * d).half().pin_memory() if pinned else torch.randn(n * heads * d).half())
    qs = [[mk(n_q, True) for _ in range(layers)] for _ in range(steps)]
    ks = [[mk(n_kv, True) for _ in range(layers)] for _ in range(steps)]
    vs = [[mk(n_kv, True) for _ in range(layers)] for _ in range(steps)]
    outs = [[(torch.empty(n * n_q * d).half().pin_memory() if (t + l) % 7 else torch.empty(n * n_q * d).half())
             for l in range(layers)] for t in range(steps)]
    for t in range(steps):
        g.begin_step(gs, [1] * n)
        for l in range(layers):
            g.attention_host_async(l, qs[t][l], ks[t][l], vs[t][l], outs[t][l], 0.09)
    g.host_sync()
    assert g.device_status() == 0
    for s_ in gs:
        assert s_.popn(steps) == steps
    for t in range(steps):
        g.begin_step(gs, [1] * n)
        for l in range(layers):
            ref = g.attention(l, qs[t][l].cuda(), ks[t][l].cuda(), vs[t][l].cuda(), 0.09).cpu()
            assert torch.equal(outs[t][l], ref), (t, l)
    assert g.device_status() == 0


@pytest.mark.parametrize("n_q,n_kv,chunk,window", [(32, 8, 512, None), (28, 4, 256, None), (28, 4, 256, 2500)])
def test_chunk_items_of_a_short_last_wave_are_cut_along_kv(n_q, n_kv, chunk, window):
    # One prompt in chunks: 64 (or 32) work items per launch on 148 SMs, so the two-tile kernel cuts every
    # item into 2 (or 4) K/V slices once the context is long enough, and the last slice to finish merges
    # them.  Checked against the oracle at every chunk; then again with the cutting switched off, which must
    # give the same numbers to within the rounding of a different summation order.
    outs = []
    for max_parts in (4, 1):
        p = Pair(1, n_q, n_kv, 128, 8192, num_pages=400, seed=77, shuffle_free_list=True)
        p.g.set_chunk_split(max_parts)
        s_ = p.new_seq()
        last = None
        for _ in range(4608 // chunk):
            last = p.step([s_], [chunk], window=window)
        outs.append(np.asarray(last[0], np.float32))
        p.assert_state_equal(pages="used")
        assert p.g.device_status() == 0
    np.testing.assert_allclose(outs[0], outs[1], atol=2e-3, rtol=1e-2)


def test_one_long_sequence_is_cut_into_many_parts():
    # a single 20 000-token sequence: every (kv head) segment is split over dozens of CTAs, so the
    # ticket merge runs with far more than eight partials
    from combsengine_b200 import KVArena
    from oracle import OracleArena
    n_q, n_kv, d, L = 28, 4, 128, 20000
    rng = np.random.default_rng(77)
    g = KVArena(1, n_q, n_kv, d, L + 64, num_pages=1300)
    o = OracleArena(1, n_kv, d, L + 64, num_pages=1300, rolling=False, dtype="f16")
    perm = rng.permutation(1300)
    g.set_free_list(perm); o.set_free_list(perm)
    gs, os_ = g.new_seq(), o.new_seq()
    k = rng.standard_normal((n_kv, L, d)).astype(np.float16)
    v = rng.standard_normal((n_kv, L, d)).astype(np.float16)
    g.begin_step([gs], [L])
    g.append(0, torch.from_numpy(k.reshape(-1)).cuda(), torch.from_numpy(v.reshape(-1)).cuda())
    o.batch_begin([os_], [L])
    os_.append_only(0, k, v, 0)
    for step, window in enumerate([None, None, 4000]):
        q, k1, v1 = (rng.standard_normal((h, 1, d)).astype(np.float16) for h in (n_q, n_kv, n_kv))
        g.begin_step([gs], [1])
        got = g.attention(0, *(torch.from_numpy(x.reshape(-1)).cuda() for x in (q, k1, v1)), d ** -0.5, window).cpu().numpy()
        o.batch_begin([os_], [1])
        ref = o.batch_layer([os_], [1], 0, q.reshape(-1), k1.reshape(-1), v1.reshape(-1), n_q, d ** -0.5, window)
        assert_attention_close(got, ref, f"long sequence step {step}")
    assert g.device_status() == 0


def test_empty_step_smallest_window_and_exact_capacity():
    from combsengine_b200 import CbkvError
    p = Pair(1, 8, 2, 64, 48, seed=13)
    from combsengine_b200.kv import launch_count
    before = launch_count()
    p.g.begin_step([], [])                      # an empty step is legal and launches nothing
    e = torch.empty(0, dtype=torch.float16, device="cuda")
    assert p.g.attention(0, e, e, e, 0.125).numel() == 0
    assert launch_count() == before
    s = p.new_seq()
    p.step([s], [30], window=2)                 # the smallest window: each query sees itself and one key before
    for _ in range(17):
        p.step([s], [1], window=2)
    assert s[0].seq_len() == 47
    p.step([s], [1])                            # exactly max_seq_len tokens
    assert s[0].seq_len() == 48 and s[0].pages_used() == 3
    with pytest.raises(CbkvError, match="capacity exceeded: 49 > 48"):
        p.g.begin_step([s[0]], [1])
    assert s[0].seq_len() == 48
    p.assert_state_equal()
