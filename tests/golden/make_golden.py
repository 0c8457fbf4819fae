"""Regenerates the golden fixtures in this folder from the CPU oracle.

    python tests/golden/make_golden.py

The reference (Rust on un-vendored crates) cannot be imported or run here, so the
fixtures are outputs of the oracle — which is itself pinned to the reference's
known-answer tests — on inputs from the reference's own deterministic generators
(`kv_tok` / `q_tok`, kv.rs:863-882, and the xorshift64 stream of tests/attn_cliff.rs:28-45).
Inputs are regenerated from those generators by the tests; only outputs and integer
state are stored.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import OracleArena  # noqa: E402


def xorshift_data(n, seed):  # tests/attn_cliff.rs:28-45
    x, m = int(seed | 1), (1 << 64) - 1
    out = np.empty(n, dtype=np.float32)
    for i in range(n):
        x ^= (x << 13) & m
        x ^= x >> 7
        x ^= (x << 17) & m
        out[i] = np.float32(np.float32((x >> 40) & 0xFFFFFFFF) / np.float32(1 << 24) * np.float32(2.0) - np.float32(1.0))
    return out


def smollm_case():
    """SmolLM2 geometry (9/3/64, scale 0.125): a 100-token chunk, then 20 decode steps, popn(7), 5 more steps."""
    n_q, n_kv, d, scale = 9, 3, 64, 0.125
    total = 100 + 20 + 5
    q = xorshift_data(n_q * total * d, 11).reshape(n_q, total, d).astype(np.float16)
    k = xorshift_data(n_kv * total * d, 22).reshape(n_kv, total, d).astype(np.float16)
    v = xorshift_data(n_kv * total * d, 33).reshape(n_kv, total, d).astype(np.float16)
    perm = np.random.default_rng(64).permutation(64)
    plan = [(0, 100)] + [(100 + i, 1) for i in range(20)] + [("popn", 7)] + [(113 + i, 1) for i in range(5)]
    return dict(n_q=n_q, n_kv=n_kv, d=d, scale=scale, q=q, k=k, v=v, perm=perm, plan=plan, max_seq_len=1024)


def run_oracle(case):
    a = OracleArena(1, case["n_kv"], case["d"], case["max_seq_len"], dtype="f16")
    a.set_free_list(case["perm"])
    s = a.new_seq()
    outs, cursor = [], 0
    for step in case["plan"]:
        if step[0] == "popn":
            assert s.popn(step[1]) == step[1]
            continue
        pos, n = step
        sl = slice(cursor, cursor + n)
        outs.append(s.attention(0, case["q"][:, sl], case["k"][:, sl], case["v"][:, sl], pos, case["scale"]).reshape(case["n_q"], n, case["d"]))
        cursor += n
    state = dict(table=s.block_table(), free=a.free_list(), seq_len=np.int64(s.seq_len()))
    pages_k = np.stack([a.page(0, int(p))[0] for p in s.block_table()])
    pages_v = np.stack([a.page(0, int(p))[1] for p in s.block_table()])
    return np.concatenate(outs, axis=1), state, pages_k, pages_v


if __name__ == "__main__":
    out, state, pk, pv = run_oracle(smollm_case())
    np.savez_compressed(os.path.join(HERE, "smollm2_chunk_decode_popn.npz"), out=out.view(np.uint16), table=state["table"],
                        free=state["free"], seq_len=state["seq_len"], pages_k=pk.view(np.uint16), pages_v=pv.view(np.uint16))
    print("wrote", os.path.join(HERE, "smollm2_chunk_decode_popn.npz"), out.shape)
