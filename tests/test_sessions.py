"""Session table, prefix reuse and speculative rollback: the library's host logic against the
restatement of combs-runtime/src/engine.rs (CPU only: bookkeeping needs no device)."""
import json

import numpy as np
import pytest

from combsengine_b200 import CbkvError, KVArena
from combsengine_b200 import sessions as S
from oracle import OracleArena
from oracle import sessions_oracle as O


def test_common_prefix_cases_of_the_reference():   # engine.rs:1786-1794
    cases = [([1, 2, 3], [1, 2, 3], 3), ([1, 2, 3], [1, 2, 4], 2), ([1, 2], [1, 2, 3, 4], 2), ([1, 2, 3, 4], [1, 2], 2),
             ([1], [2], 0), ([], [1], 0), ([1], [], 0)]
    for a, b, n in cases:
        assert O.common_prefix(a, b) == n
    # the library: a session whose history is `a`, then a prompt `b`; lcp = min(common, len(b) - 1)
    for a, b, n in cases:
        if not a or not b:
            continue
        arena = KVArena(1, 2, 1, 64, 64, num_pages=8)
        ss = S.SessionSet(arena)
        s, lcp = ss.acquire("k", a)
        assert lcp == 0
        arena.begin_step_host_only([s], [len(a)])
        ss.release("k", s, a)
        s2, lcp = ss.acquire("k", b)
        assert lcp == min(n, len(b) - 1)
        assert s2.seq_len() == lcp
        ss.close()


def _pair(max_sessions=4, windows=None, layers=2, pages=64, max_len=256):
    g = KVArena(layers, 4, 2, 64, max_len, num_pages=pages, windows=windows)
    o = OracleArena(layers, 2, 64, max_len, num_pages=pages, windows=windows, rolling=windows is not None, dtype="f16")
    return g, o, S.SessionSet(g, max_sessions), O.OracleSessionSet(o, max_sessions)


def _same_state(g, o, gs, os_):
    assert gs.seq_len() == os_.seq_len()
    assert list(gs.block_table()) == list(os_.block_table())
    assert list(g.free_list()) == list(o.free_list())


def test_random_generations_match_the_restatement():
    rng = np.random.default_rng(42)
    g, o, gset, oset = _pair()
    keys = ["", "alice", "bob", "carol", "dave", "erin"]
    histories: dict[str, list] = {}
    for it in range(300):
        key = keys[rng.integers(len(keys))]
        base = histories.get(key, [])
        if base and rng.random() < 0.7:      # continue a conversation: shared prefix, maybe a divergent tail
            cut = int(rng.integers(0, len(base) + 1))
            prompt = base[:cut] + [int(x) for x in rng.integers(0, 50, size=rng.integers(1, 12))]
        else:
            prompt = [int(x) for x in rng.integers(0, 50, size=rng.integers(1, 30))]
        prompt = prompt[:120]
        reuse = rng.random() < 0.9
        gs, glcp = gset.acquire(key, prompt, reuse)
        os_, olcp = oset.acquire(key, prompt, reuse)
        assert glcp == olcp, f"iteration {it}"
        _same_state(g, o, gs, os_)
        # prefill the suffix, then decode a few tokens, some of them through speculative rounds
        g.begin_step_host_only([gs], [len(prompt) - glcp]); o.batch_begin([os_], [len(prompt) - olcp])
        decoded = []
        for _ in range(int(rng.integers(0, 8))):
            if rng.random() < 0.4:
                k = int(rng.integers(1, 5))
                draft = [int(x) for x in rng.integers(0, 3, size=k)]
                argmax = [int(x) for x in rng.integers(0, 3, size=k + 1)]
                g.begin_step_host_only([gs], [k + 1]); o.batch_begin([os_], [k + 1])
                ga = S.spec_verify_rollback(gs, draft, argmax)
                oa = O.spec_verify_rollback(os_, draft, argmax)
                assert ga == oa
                decoded += [7] + draft[:ga[0]]
            else:
                g.begin_step_host_only([gs], [1]); o.batch_begin([os_], [1])
                decoded.append(int(rng.integers(0, 50)))
        hist = prompt + decoded
        _same_state(g, o, gs, os_)
        assert gs.seq_len() == len(hist)
        gset.release(key, gs, hist, reuse); oset.release(key, os_, hist, reuse)
        if reuse:
            histories[key] = hist
        assert len(gset) == len(oset.map) <= 4 and gset.evictions == oset.evictions
        assert list(g.free_list()) == list(o.free_list())
        for k2 in keys:
            want = len(oset.map[k2]["history"]) if k2 in oset.map else None
            assert gset.history_len(k2) == want
    assert gset.evictions > 0
    assert gset.clear_all() == oset.clear_all()
    assert g.num_free_pages() == g.num_pages and list(g.free_list()) == list(o.free_list())


def test_refused_rollback_starts_fresh():
    # a sliding layer past its window makes popn refuse (kv.rs:812-816): the session is rebuilt, never
    # continued on divergent state (engine.rs:1275-1284)
    g, o, gset, oset = _pair(windows=[None, 8])
    hist = list(range(40))
    for st, arena in ((gset, g), (oset, o)):
        s, lcp = st.acquire("w", hist)
        (arena.begin_step_host_only if arena is g else arena.batch_begin)([s], [40])
        st.release("w", s, hist)
    gs, glcp = gset.acquire("w", hist[:20] + [99])
    os_, olcp = oset.acquire("w", hist[:20] + [99])
    assert glcp == olcp == 0 and gs.seq_len() == 0
    assert list(g.free_list()) == list(o.free_list())


def test_release_checks_the_history_and_stats_json_has_the_reference_fields():
    g, o, gset, oset = _pair()
    s, _ = gset.acquire(None, [1, 2, 3])
    g.begin_step_host_only([s], [3])
    with pytest.raises(CbkvError, match="does not mirror"):
        gset.release(None, s, [1, 2])
    gset.release(None, s, [1, 2, 3])
    s2, _ = gset.acquire('we"ird', [5] * 20)
    g.begin_step_host_only([s2], [20])
    gset.release('we"ird', s2, [5] * 20)
    kv = gset.stats()
    assert kv["kind"] == "paged" and kv["quantized"] is False and kv["page_size"] == 16 and kv["max_sessions"] == 4
    assert kv["page_bytes"] == g.page_bytes() == 16 * 2 * 64 * 2 * 2 * 2      # engine.rs:489-496
    assert kv["arena_bytes"] == 64 * kv["page_bytes"] and kv["bytes_per_token"] == kv["page_bytes"] // 16
    ids = [x["id"] for x in kv["sessions"]]
    assert ids == ["(anonymous)", 'we"ird']
    p = kv["sessions"][1]["pages"]
    assert set(p) == {"used", "free", "total", "page_size", "seq_len", "kv_bytes", "layers_materialized", "layers_total",
                      "layers_sliding"}
    assert p["used"] == 2 and p["seq_len"] == 20 and p["kv_bytes"] == 2 * kv["page_bytes"] and p["free"] == 64 - 3
    assert kv["sessions"][0]["history_tokens"] == 3


def test_partial_speculative_pop_is_an_error():
    g = KVArena(2, 4, 2, 64, 256, num_pages=32, windows=[None, 8])
    s = g.new_seq()
    g.begin_step_host_only([s], [30])
    with pytest.raises(CbkvError, match="speculative rollback popped 0 of 2 rows"):
        S.spec_verify_rollback(s, [1, 2, 3], [1, 9, 9, 9])


@pytest.mark.gpu
def test_prefix_reuse_and_speculative_rollback_on_the_device():
    """Two conversations over one arena with evictions, prefix reuse and speculative rounds; every
    forward pass is checked against the oracle and the pages are bit-exact at the end."""
    from kvcase import Pair
    p = Pair(2, 8, 2, 128, 512, num_pages=96, seed=11, shuffle_free_list=True)
    gset, oset = S.SessionSet(p.g, 2), O.OracleSessionSet(p.o, 2)
    rng = np.random.default_rng(5)
    hist = {}
    for it in range(8):
        key = ["a", "b", "c"][it % 3]
        base = hist.get(key, [])
        prompt = (base[:max(0, len(base) - 5)] + [int(x) for x in rng.integers(0, 99, size=40)])[:300]
        gs, glcp = gset.acquire(key, prompt)
        os_, olcp = oset.acquire(key, prompt)
        assert glcp == olcp
        pair = (gs, os_)
        p.seqs = [q for q in p.seqs if q[0]._h is not None]
        if pair not in p.seqs:
            p.seqs.append(pair)
        p.step([pair], [len(prompt) - glcp])
        decoded = []
        for r in range(3):
            draft = [1, 2, 3]
            argmax = [1, 2, 9, 9] if r % 2 == 0 else [4, 4, 4, 4]
            p.step([pair], [len(draft) + 1])
            acc = S.spec_verify_rollback(gs, draft, argmax)
            assert acc == O.spec_verify_rollback(os_, draft, argmax)
            decoded += [7] + draft[:acc[0]]
            p.step([pair], [1])
            decoded.append(8)
        h = prompt + decoded
        gset.release(key, gs, h); oset.release(key, os_, h)
        hist[key] = h
        p.seqs = [q for q in p.seqs if q[0]._h is not None]
    assert gset.evictions == oset.evictions > 0
    p.assert_state_equal(pages="used")
