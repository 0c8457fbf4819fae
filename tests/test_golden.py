"""Committed golden fixtures (tests/golden/, made by make_golden.py from the oracle on the
reference's own deterministic input generators): the oracle must keep reproducing them
bit for bit, and the CUDA path must match them (state exactly, attention within tolerance)."""
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_golden  # noqa: E402

FIXTURE = os.path.join(HERE, "golden", "smollm2_chunk_decode_popn.npz")


def test_oracle_reproduces_the_golden_fixture_bit_for_bit():
    g = np.load(FIXTURE)
    out, state, pk, pv = make_golden.run_oracle(make_golden.smollm_case())
    assert np.array_equal(out.view(np.uint16), g["out"])
    assert list(state["table"]) == list(g["table"]) and list(state["free"]) == list(g["free"])
    assert int(state["seq_len"]) == int(g["seq_len"]) == 118
    assert np.array_equal(pk.view(np.uint16), g["pages_k"]) and np.array_equal(pv.view(np.uint16), g["pages_v"])


@pytest.mark.gpu
def test_cuda_path_matches_the_golden_fixture():
    import torch
    from combsengine_b200 import KVArena
    from kvcase import assert_attention_close

    g = np.load(FIXTURE)
    c = make_golden.smollm_case()
    a = KVArena(1, c["n_q"], c["n_kv"], c["d"], c["max_seq_len"])
    a.set_free_list(c["perm"])
    s = a.new_seq()
    outs, cursor = [], 0
    for step in c["plan"]:
        if step[0] == "popn":
            assert s.popn(step[1]) == step[1]
            continue
        pos, n = step
        sl = slice(cursor, cursor + n)
        a.begin_step([s], [n], [pos])
        dev = lambda x: torch.from_numpy(np.ascontiguousarray(x[:, sl]).reshape(-1)).cuda()
        outs.append(a.attention(0, dev(c["q"]), dev(c["k"]), dev(c["v"]), c["scale"]).cpu().numpy().reshape(c["n_q"], n, c["d"]))
        cursor += n
    assert a.device_status() == 0
    got = np.concatenate(outs, axis=1)
    assert_attention_close(got, g["out"].view(np.float16), "golden attention outputs")
    assert list(s.block_table()) == list(g["table"]) and list(a.free_list()) == list(g["free"]) and s.seq_len() == int(g["seq_len"])
    for i, pg in enumerate(s.block_table()):
        gk, gv = a.export_page(0, int(pg))
        assert np.array_equal(gk, g["pages_k"][i]) and np.array_equal(gv, g["pages_v"][i])
