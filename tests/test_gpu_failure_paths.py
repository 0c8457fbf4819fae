"""The kernels' failure paths, driven without faulting or hanging anything (needs a B200).

A kernel never traps: a block-table entry outside the arena is replaced by page 0 for reading and
skipped for writing, a wait that runs out makes the warp give up, and both are reported in the
arena's status word.  Here the bad entry comes from a caller-owned block table (the library's own
tables cannot hold one), and the wait runs out because a test hook makes the producer withhold
one tile's copy while the wait limit is lowered to a millisecond.  Both launches return normally
and the next step computes correct results.
"""
import numpy as np
import pytest
import torch

from kvcase import Pair

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_sets_the_status_word_and_the_next_step_is_correct():
    p = Pair(2, 28, 4, 128, 2048, num_pages=300, shuffle_free_list=True, seed=77)
    seqs = [p.new_seq() for _ in range(4)]
    p.step(seqs, [200, 333, 64, 500], check=False)
    p.step(seqs, [1, 1, 1, 1])                      # a clean decode step first
    g = p.g
    g.debug_set_wait_limit(wait_us=1000, fault_tile=3)   # CTA 0 never receives its fourth tile
    gs = [s[0] for s in seqs]
    g.begin_step(gs, [1] * 4, [s.seq_len() for s in gs])
    p.o.batch_begin([s[1] for s in seqs], [1] * 4)
    mk = lambda h: np.concatenate([p.rand(h, 1).reshape(-1) for _ in seqs])
    for layer in range(2):
        q, k, v = mk(28), mk(4), mk(4)
        g.attention(layer, *(torch.from_numpy(x).cuda() for x in (q, k, v)), 128 ** -0.5)
        p.o.batch_layer([s[1] for s in seqs], [1] * 4, layer, q, k, v, 28, 128 ** -0.5)  # keeps the oracle in step
    torch.cuda.synchronize()                         # the launches came back
    assert g.device_status() & 2, "ST_WAIT_TIMEOUT expected"
    assert g.device_status() == 0, "reading the word clears it"
    g.debug_set_wait_limit(wait_us=100000, fault_tile=-1)
    # The step that failed left undefined rows in the pages of the tokens it appended, so the
    # sequences are rolled back over them and the tokens written again by a healthy step.
    for a, b in seqs:
        assert a.popn(1) == 1 and b.popn(1) == 1
    for _ in range(3):
        p.step(seqs, [1, 1, 1, 1])                   # checked against the oracle inside
    p.assert_state_equal(pages="used")


def test_ticket_counters_are_clean_after_a_failed_launch():
    # The failed launch may leave per-segment tickets behind.  The status word is deliberately not read
    # before the next step (reading it also clears the tickets): begin_step alone must restore them.
    from kvcase import assert_attention_close

    p = Pair(1, 8, 4, 128, 4096, num_pages=600, shuffle_free_list=True, seed=78,
             tuning=dict(max_ctas=5))               # few CTAs: every segment is cut across CTAs
    seqs = [p.new_seq() for _ in range(2)]
    p.step(seqs, [900, 700], check=False)
    g, gs, os_ = p.g, [s[0] for s in seqs], [s[1] for s in seqs]

    def raw_step():
        g.begin_step(gs, [1, 1], [s.seq_len() for s in gs])
        p.o.batch_begin(os_, [1, 1])
        q, k, v = (np.concatenate([p.rand(h, 1).reshape(-1) for _ in seqs]) for h in (8, 4, 4))
        out = g.attention(0, *(torch.from_numpy(x).cuda() for x in (q, k, v)), 0.09).cpu().numpy()
        return out, p.o.batch_layer(os_, [1, 1], 0, q, k, v, 8, 0.09)

    g.debug_set_wait_limit(wait_us=1000, fault_tile=1)
    raw_step()
    g.debug_set_wait_limit(wait_us=100000, fault_tile=-1)
    for a, b in seqs:
        assert a.popn(1) == 1 and b.popn(1) == 1
    for i in range(3):
        got, ref = raw_step()
        assert_attention_close(got, ref, f"step {i} after the failed launch")
    assert g.device_status() & 2   # the word still remembers the failed launch; now it is read and cleared
    assert g.device_status() == 0
    p.assert_state_equal(pages="used")
