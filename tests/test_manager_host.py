"""Host logic through the C ABI, no GPU: the manager against the reference's
known-answer tests (kv.rs:1075-1192) and against the oracle on random histories,
the decode work split, and the boundary itself (symbols, loud failure)."""
import ctypes as C
import os
import re

import numpy as np
import pytest
import torch

from combsengine_b200 import CbkvError, KVArena, _lib
from oracle import OracleArena

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def arena(max_seq_len=64, page_size=16, layers=2, num_pages=0, windows=None, **kw):
    return KVArena(layers, 4, 2, 64, max_seq_len, page_size, num_pages, windows, **kw)


def grow(a, s, total):  # the reference tests' grow() helper, kv.rs:1134-1137
    a.begin_step_host_only([s], [total - s.seq_len()])


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "combs_kv.h")).read()
    declared = set(re.findall(r"\b(cbkv_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    lib = C.CDLL(_lib.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} declared in include/combs_kv.h but not exported"
    assert declared == set(_lib.PROTOTYPES), "ctypes prototypes and header disagree"


def test_allocator_order_lifo_reset():  # kv.rs:1075-1107
    a = arena(48)
    s = a.new_seq()
    assert a.num_free_pages() == 3
    grow(a, s, 48)
    assert list(s.block_table()) == [0, 1, 2] and a.num_free_pages() == 0
    with pytest.raises(CbkvError, match="capacity exceeded"):
        grow(a, s, 49)
    assert s.popn(48) == 48
    assert list(a.free_list()) == [2, 1, 0]  # pushed in table.pop() order
    grow(a, s, 32)
    assert list(s.block_table()) == [0, 1]
    s.reset()
    assert a.num_free_pages() == 3 and list(a.free_list()) == [2, 1, 0]


def test_exhaustion_is_all_or_nothing():  # kv.rs:552-555
    a = arena(64, num_pages=3)
    s, t = a.new_seq(), a.new_seq()
    grow(a, s, 32)
    with pytest.raises(CbkvError, match="page allocator exhausted") as e:
        a.begin_step_host_only([s, t], [1, 17])
    assert e.value.code == -3
    assert s.seq_len() == 32 and t.seq_len() == 0 and a.num_free_pages() == 1


@pytest.mark.parametrize("n,pages", [(16, 1), (17, 2), (1, 1)])
def test_num_pages_rounds_up(n, pages):  # kv.rs:1109-1114
    assert arena(n).num_free_pages() == pages


def test_popn_frees_only_fully_unused_pages():  # kv.rs:1139-1160
    a = arena()
    c = a.new_seq()
    grow(a, c, 40)
    assert c.pages_used() == 3 and a.num_free_pages() == 1
    c.popn(9)
    assert (c.seq_len(), c.pages_used(), a.num_free_pages()) == (31, 2, 2)
    c.popn(15)
    assert c.pages_used() == 1
    c.popn(1)
    assert c.pages_used() == 1
    assert c.popn(1000) == 15
    assert (c.seq_len(), c.pages_used(), a.num_free_pages()) == (0, 0, 4)


def test_popn_boundary_and_regrowth_and_reset():  # kv.rs:1162-1192
    a = arena()
    c = a.new_seq()
    grow(a, c, 32)
    c.popn(16)
    assert c.pages_used() == 1 and a.num_free_pages() == 3
    c.popn(16)
    assert c.pages_used() == 0 and a.num_free_pages() == 4
    grow(a, c, 40)
    freed = c.block_table()[2]
    c.popn(9)
    grow(a, c, 33)
    assert c.pages_used() == 3 and a.num_free_pages() == 1 and c.block_table()[2] == freed
    c.reset()
    assert (c.seq_len(), c.pages_used(), a.num_free_pages()) == (0, 0, 4)


def test_errors_carry_the_reference_messages():
    a = arena(8, 4)
    s = a.new_seq()
    with pytest.raises(CbkvError, match=r"paged cache capacity exceeded: 9 > 8") as e:  # tests/kv_cache.rs:167-173
        a.begin_step_host_only([s], [9])
    assert e.value.code == -2 and s.seq_len() == 0
    with pytest.raises(CbkvError, match="dense contiguous appends") as e:  # kv.rs:671-674
        a.begin_step_host_only([s], [2], [3])
    assert e.value.code == -1
    with pytest.raises(CbkvError, match="sliding window must be >= 2, got 1"):  # kv.rs:514-516
        arena(windows=[1, None])
    with pytest.raises(CbkvError, match="one window entry per layer"):  # kv.rs:513
        arena(windows=[4])


def test_sliding_popn_refusal_rule():  # kv.rs:812-816, 1061-1073
    a = arena(64, windows=[4, None])
    s = a.new_seq()
    grow(a, s, 3)
    assert s.popn(1) == 1  # nothing evicted yet (seq_len <= w - 1)
    grow(a, s, 6)
    assert s.popn(1) == 0 and s.seq_len() == 6
    assert s.popn(0) == 0
    b = arena(64, windows=[4, None], sliding_popn_refuses=False)
    t = b.new_seq()
    grow(b, t, 6)
    assert t.popn(1) == 1


def test_page_stats_fields():  # kv.rs:535-546
    a = arena(64, windows=[None, 8])
    s = a.new_seq()
    grow(a, s, 20)
    st = s.page_stats()
    assert (st.pages_used, st.pages_free, st.num_pages, st.page_size, st.seq_len) == (2, 2, 4, 16, 20)
    assert (st.layers_materialized, st.layers_total, st.layers_sliding) == (0, 2, 0)
    assert a.page_bytes() == 16 * 2 * 64 * 2 * 2 * 2  # engine.rs:475-498


def test_prefix_sharing_refcounts_and_guards():
    a = arena(256, num_pages=16)
    p = a.new_seq()
    grow(a, p, 40)
    with pytest.raises(CbkvError, match="whole pages"):
        p.fork_prefix(20)
    c = p.fork_prefix(32)
    assert c.seq_len() == 32 and list(c.block_table()) == list(p.block_table()[:2])
    assert [a.refcount(int(x)) for x in p.block_table()] == [2, 2, 1]
    grow(a, c, 33)  # the child's first append takes a fresh page
    assert c.block_table()[2] not in p.block_table()
    assert c.popn(10) == 0  # would end inside a shared page
    assert c.popn(1) == 1 and c.pages_used() == 2
    free_before = a.num_free_pages()
    c.close()  # shared pages stay with the parent
    assert a.num_free_pages() == free_before
    assert [a.refcount(int(x)) for x in p.block_table()] == [1, 1, 1]


def random_history(seed, rolling=False):
    """The same random allocate/append/popn/fork/destroy/reset history on the manager and the oracle."""
    rng = np.random.default_rng(seed)
    pages = 96
    a = KVArena(2, 4, 2, 64, 400, 16, pages, sliding_popn_refuses=False)
    o = OracleArena(2, 2, 64, 400, 16, pages, rolling=False, dtype="f16")
    perm = rng.permutation(pages)
    a.set_free_list(perm)
    o.set_free_list(perm)
    seqs = []
    for step in range(300):
        op = rng.integers(0, 10)
        if op <= 1 and len(seqs) < 10:
            seqs.append((a.new_seq(), o.new_seq()))
        elif op <= 5 and seqs:
            idx = rng.permutation(len(seqs))[: rng.integers(1, len(seqs) + 1)]
            new = [int(rng.integers(1, 40)) for _ in idx]
            ok = True
            try:
                a.begin_step_host_only([seqs[i][0] for i in idx], new)
            except CbkvError as e:
                ok = False
                code = e.code
            if ok:
                o.batch_begin([seqs[i][1] for i in idx], new)
            else:
                with pytest.raises(Exception):
                    o.batch_begin([seqs[i][1] for i in idx], new)
                # the oracle is not all-or-nothing across a batch; rebuild it from the manager's state
                return None if code == 0 else "diverged-on-error"
        elif op == 6 and seqs:
            i = rng.integers(len(seqs))
            n = int(rng.integers(0, 50))
            assert seqs[i][0].popn(n) == seqs[i][1].popn(n)
        elif op == 7 and seqs:
            i = rng.integers(len(seqs))
            n = (seqs[i][0].seq_len() // 16) * 16
            if n and len(seqs) < 10:
                n = int(rng.integers(1, n // 16 + 1)) * 16
                seqs.append((seqs[i][0].fork_prefix(n), seqs[i][1].fork_prefix(n)))
        elif op == 8 and seqs:
            i = rng.integers(len(seqs))
            s, t = seqs.pop(i)
            s.close(); t.close()
        elif op == 9 and seqs and rng.integers(4) == 0:
            i = rng.integers(len(seqs))
            seqs[i][0].reset(); seqs[i][1].reset()
        assert list(a.free_list()) == list(o.free_list()), step
        for s, t in seqs:
            assert s.seq_len() == t.seq_len()
            assert list(s.block_table()) == list(t.block_table())
        for pg in range(pages):
            assert a.refcount(pg) == o.refcount(pg)
    return "done"


@pytest.mark.parametrize("seed", range(6))
def test_manager_matches_oracle_on_random_histories(seed):
    random_history(seed)


@pytest.mark.parametrize("window,n_ctas,tail_pct,min_item", [(0, 1, -1, -1), (0, 7, -1, -1), (0, 148, -1, -1), (0, 148, 40, 4),
                                                              (0, 296, 25, 0), (0, 5000, -1, -1), (100, 13, -1, -1),
                                                              (1024, 148, -1, 2), (17, 64, -1, -1)])
def test_decode_plan_covers_every_page_once(window, n_ctas, tail_pct, min_item):
    rng = np.random.default_rng(window + n_ctas)
    a = KVArena(1, 28, 4, 128, 5000, 16, 20000)
    seqs = [a.new_seq() for _ in range(24)]
    lens = [int(x) for x in rng.integers(1, 4100, len(seqs))]
    lens[0], lens[1], lens[2] = 2, 16, 17  # lengths after the decode step
    a.begin_step_host_only(seqs, [n - 1 for n in lens])   # the cached prefix
    a.begin_step_host_only(seqs, [1] * len(seqs))         # the decode step being split
    L = [s.seq_len() for s in seqs]
    pl = a.debug_decode_plan(window, n_ctas, tail_pct, min_item)
    Hkv = 4
    segs, items = pl["segs"], pl["items"]
    assert pl["n_segs"] == len(seqs) * Hkv and pl["n_items"] == pl["n_ctas"] * pl["levels"]
    sub = segs[:, 0]
    assert sub[0] == 0 and sub[-1] == pl["n_units"]
    # segments: the visible pages of every (sequence, kv head)
    tok = 0
    for b, n in enumerate(L):
        q = n - 1
        lo = max(0, q - window + 1) if window else 0
        for h in range(Hkv):
            s = b * Hkv + h
            assert segs[s, 1] == lo // 16 and segs[s, 2] == q and segs[s, 3] == tok
            assert sub[s + 1] - sub[s] == q // 16 - lo // 16 + 1
        tok += 1
    # items: non-empty, disjoint, and together exactly the units
    assert np.all(items[:, 1] > items[:, 0])
    order = np.argsort(items[:, 0], kind="stable")
    srt = items[order]
    assert srt[0, 0] == 0 and srt[-1, 1] == pl["n_units"] and np.array_equal(srt[1:, 0], srt[:-1, 1])
    # claim order: a CTA's first item is the head of its range, and later levels never grow
    G, J = pl["n_ctas"], pl["levels"]
    size = (items[:, 1] - items[:, 0]).reshape(J, G)
    if J > 1:
        assert size[0].min() >= size[1:].max()
        assert np.all(size[1:-1].min(axis=1) + 1 >= size[2:].max(axis=1)) if J > 2 else True
    # a CTA's first item is a function of the launch totals alone (the kernel computes it instead of reading it)
    U, pct = pl["n_units"], (25 if tail_pct < 0 else tail_pct) if J > 1 else 0
    for c in range(G):
        rb, re = U * c // G, U * (c + 1) // G
        assert items[c, 0] == rb and items[c, 1] == re - (re - rb) * pct // 100
    per_range = size.sum(axis=0)
    assert per_range.max() - per_range.min() <= 1  # balanced to one page before any claiming
    # parts: every segment knows how many items touch it, and every item its place among them
    parts = 0
    for s in range(pl["n_segs"]):
        touching = [i for i in order if items[i, 0] < sub[s + 1] and items[i, 1] > sub[s]]
        assert segs[s, 4] == len(touching)
        if len(touching) > 1:
            assert segs[s, 5] == parts
            parts += len(touching)
        else:
            assert segs[s, 5] == -1
        for rank, i in enumerate(touching):
            if sub[s] <= items[i, 0] < sub[s + 1]:
                assert items[i, 2] == s and items[i, 3] == rank
            else:
                assert rank == 0  # an item that runs into a segment from before it is that segment's part 0
    assert parts == pl["n_parts"]


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the behaviour on a machine without a GPU")
def test_compute_fails_loudly_without_a_gpu():
    a = arena()
    s = a.new_seq()
    lib = _lib.load()
    hs = (C.c_void_p * 1)(s._h)
    nt = (C.c_int64 * 1)(1)
    rc = lib.cbkv_begin_step(a._h, hs, nt, None, 1, None)
    assert rc == -5 and b"no CPU path" in lib.cbkv_last_error()
    assert s.seq_len() == 0  # nothing advanced
    assert lib.cbkv_attention(a._h, 0, None, None, None, None, 1.0, 0, None) == -6  # no step begun


def test_empty_step_changes_nothing():
    a = KVArena(2, 8, 2, 64, 64, num_pages=8)
    s = a.new_seq()
    a.begin_step_host_only([s], [20])
    free = a.num_free_pages()
    a.begin_step_host_only([], [])
    assert s.seq_len() == 20 and s.pages_used() == 2 and a.num_free_pages() == free
