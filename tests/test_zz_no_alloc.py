"""The allocation-free decode entry point against the regular one (needs a B200).

``cbkv_decode_attention_static`` exists for callers that are not allowed to
allocate device memory while they run; it keeps the kernel's working memory in a
fixed array inside the library.  This file is collected last on purpose: if it
fails, a run that stops at the first failure has already run everything else.
The same pages are given to both entry points and two calls are made in a row,
because the second call reuses whatever the first left in the shared array.  The
output is also compared with the CPU oracle directly, and the entry point's own
status word (which lives in the shared array) is read after every call.
"""
import numpy as np
import pytest
import torch

from kvcase import assert_attention_close

pytestmark = pytest.mark.gpu


def test_static_decode_matches_regular_entry_point_twice_in_a_row():
    from combsengine_b200 import KVArena
    from combsengine_b200.kv import decode_attention_static, static_status
    from oracle import OracleContiguous

    n_q, n_kv, d, num_pages = 28, 4, 128, 600
    rng = np.random.default_rng(0xA110C)
    # no length is a multiple of 16, so the decoded token stays in the last prefix page
    prefix = [int(x) for x in rng.integers(40, 1500, 6)]
    prefix = [n + 1 if n % 16 == 0 or (n + 1) % 16 == 0 else n for n in prefix]
    perm = rng.permutation(num_pages)

    # regular path: library-owned arena, prefix appended, then one decode step
    arena = KVArena(1, n_q, n_kv, d, 2048, num_pages=num_pages)
    arena.set_free_list(perm)
    seqs = [arena.new_seq() for _ in prefix]
    kpre = [rng.standard_normal((n_kv, n, d)).astype(np.float16) for n in prefix]
    vpre = [rng.standard_normal((n_kv, n, d)).astype(np.float16) for n in prefix]
    knew = [rng.standard_normal((n_kv, 1, d)).astype(np.float16) for _ in prefix]
    vnew = [rng.standard_normal((n_kv, 1, d)).astype(np.float16) for _ in prefix]
    pk = lambda xs: torch.from_numpy(np.concatenate([x.reshape(-1) for x in xs])).cuda()
    arena.begin_step(seqs, prefix)
    arena.append(0, pk(kpre), pk(vpre))
    arena.begin_step(seqs, [1] * len(seqs))
    arena.append(0, pk(knew), pk(vnew))
    tables = [s.block_table() for s in seqs]
    lens = [s.seq_len() for s in seqs]

    # the caller-owned copy of the same pages, in the library's page layout
    # [page][kv head][slots 0-7 / 8-15][K, V][slot within the half][d]
    pages = torch.zeros(num_pages, n_kv, 2, 2, 8, d, dtype=torch.float16)
    for b, tbl in enumerate(tables):
        kk = np.concatenate([kpre[b], knew[b]], axis=1)
        vv = np.concatenate([vpre[b], vnew[b]], axis=1)
        for t in range(lens[b]):
            slot = t % 16
            pages[int(tbl[t // 16]), :, slot // 8, 0, slot % 8] = torch.from_numpy(kk[:, t])
            pages[int(tbl[t // 16]), :, slot // 8, 1, slot % 8] = torch.from_numpy(vv[:, t])
    pages = pages.cuda()
    stride = max(len(t) for t in tables)
    bt = torch.zeros(len(seqs), stride, dtype=torch.int32)
    for b, tbl in enumerate(tables):
        bt[b, : len(tbl)] = torch.from_numpy(tbl.astype(np.int32))
    bt = bt.cuda()

    out = torch.empty(len(seqs) * n_q * d, dtype=torch.float16, device="cuda")
    for call, (scale, window) in enumerate([(d ** -0.5, None), (0.07, 200)]):
        qs = [rng.standard_normal((n_q, 1, d)).astype(np.float16) for _ in prefix]
        q = pk(qs)
        ref = arena.paged_attention(0, q, scale, window).cpu().numpy()
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        decode_attention_static(pages, bt, lens, n_q, n_kv, d, q, out, scale, window)
        assert static_status() == 0, "the static entry point's own status word"
        if call > 0:  # the first call makes the driver load the module that holds the fixed array
            assert torch.cuda.mem_get_info()[0] >= free_before, "the entry point must not allocate device memory"
        got = out.cpu().numpy()
        assert_attention_close(got, ref, f"static decode vs the regular entry point, call {call}")
        # and against the oracle itself: the reference's contiguous cache fed the same tokens (kv.rs:360-415)
        want = []
        for b, n in enumerate(prefix):
            c = OracleContiguous(1, n_kv, d, dtype="f16")
            c.attention_opts(0, np.zeros((n_q, n, d), np.float16), kpre[b], vpre[b], 0, scale, window)
            want.append(c.attention_opts(0, qs[b], knew[b], vnew[b], n, scale, window).reshape(-1))
        assert_attention_close(got, np.concatenate(want), f"static decode vs the oracle, call {call}")
    assert arena.device_status() == 0


def test_static_decode_reports_a_bad_block_table_entry_in_its_own_status_word():
    # a page id outside the caller's pages: the kernel reads page 0 instead, finishes, and says so
    from combsengine_b200.kv import decode_attention_static, static_status

    n_q, n_kv, d, num_pages = 8, 2, 128, 16
    pages = torch.randn(num_pages, n_kv, 2, 2, 8, d, device="cuda").half()
    bt = torch.tensor([[3, 5, num_pages + 7, 1], [2, 4, 6, 8]], dtype=torch.int32, device="cuda")
    q = torch.randn(2 * n_q * d, device="cuda").half()
    out = decode_attention_static(pages, bt, [60, 50], n_q, n_kv, d, q)
    assert static_status() == 1  # ST_BAD_PAGE, and the word is cleared by the read
    assert static_status() == 0
    assert torch.isfinite(out.float()).all()
    bt[0, 2] = 9
    decode_attention_static(pages, bt, [60, 50], n_q, n_kv, d, q)
    assert static_status() == 0


def test_static_decode_refuses_sizes_beyond_its_working_memory():
    from combsengine_b200 import CbkvError
    from combsengine_b200.kv import decode_attention_static

    pages = torch.zeros(8, 4, 2, 2, 8, 128, dtype=torch.float16, device="cuda")
    bt = torch.zeros(129, 2, dtype=torch.int32, device="cuda")
    q = torch.zeros(129 * 28 * 128, dtype=torch.float16, device="cuda")
    with pytest.raises(CbkvError, match="too large for the static working memory"):
        decode_attention_static(pages, bt, [5] * 129, 28, 4, 128, q)
