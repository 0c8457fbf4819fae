"""KV heads sharded over two GPUs, joined by one NCCL all-gather (needs two B200s; skipped on one).

Each rank runs the real kernels on its half of the kv heads (and the matching q heads) of the same
sequences; `all_gather_heads` puts the shards together.  The result must match what one GPU computes
with all heads and what the oracle computes, within the attention tolerance (a kv-head group's attention
does not depend on the other groups, but the work split, and with it the summation order, does).
Plain NCCL only: every shard lands in local memory first.
"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q_out):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from combsengine_b200 import KVArena
        from combsengine_b200.sharding import all_gather_heads, kv_head_range
        n_q, n_kv, d, pages = 28, 4, 128, 400
        rep = n_q // n_kv
        rng = np.random.default_rng(4242)  # the same inputs on every rank
        lens = [333, 64, 1000, 17]
        perm = rng.permutation(pages)
        mk = lambda heads, n: rng.standard_normal((heads, n, d)).astype(np.float16)
        kpre, vpre = [mk(n_kv, n) for n in lens], [mk(n_kv, n) for n in lens]
        steps = [([mk(n_q, 1) for _ in lens], [mk(n_kv, 1) for _ in lens], [mk(n_kv, 1) for _ in lens]) for _ in range(3)]
        heads = kv_head_range(n_kv, rank, world)
        pk = lambda xs, sl: torch.from_numpy(np.concatenate([np.ascontiguousarray(x[sl]).reshape(-1) for x in xs])).cuda()

        def run(kv_slice, q_slice, nq, nkv):
            arena = KVArena(1, nq, nkv, d, 2048, num_pages=pages, device=rank)
            arena.set_free_list(perm)
            seqs = [arena.new_seq() for _ in lens]
            arena.begin_step(seqs, lens)
            arena.append(0, pk(kpre, kv_slice), pk(vpre, kv_slice))
            outs = []
            for q, k, v in steps:
                arena.begin_step(seqs, [1] * len(lens))
                o = arena.attention(0, pk(q, q_slice), pk(k, kv_slice), pk(v, kv_slice), d ** -0.5)
                outs.append(o.view(len(lens), nq, d))  # one token per sequence: [tokens, heads, d]
            assert arena.device_status() == 0
            return outs

        kv_sl = slice(heads.start, heads.stop)
        q_sl = slice(heads.start * rep, heads.stop * rep)
        shard = run(kv_sl, q_sl, len(heads) * rep, len(heads))
        full = [all_gather_heads(o) for o in shard]
        ok_bits = ok_oracle = True
        if rank == 0:
            from oracle import OracleArena
            from kvcase import assert_attention_close
            ref = run(slice(None), slice(None), n_q, n_kv)
            try:
                for a, b in zip(full, ref):
                    assert_attention_close(a.cpu().numpy(), b.cpu().numpy(), "head-sharded decode vs one GPU")
            except AssertionError:
                ok_bits = False
            o = OracleArena(1, n_kv, d, 2048, num_pages=pages, rolling=False, dtype="f16")
            o.set_free_list(perm)
            os_ = [o.new_seq() for _ in lens]
            cat = lambda xs: np.concatenate([x.reshape(-1) for x in xs])
            o.batch_begin(os_, lens)
            o.batch_layer(os_, lens, 0, cat([mk(n_q, n) for n in lens]), cat(kpre), cat(vpre), n_q, d ** -0.5)
            for (q, k, v), got in zip(steps, full):
                o.batch_begin(os_, [1] * len(lens))
                want = o.batch_layer(os_, [1] * len(lens), 0, cat(q), cat(k), cat(v), n_q, d ** -0.5)
                try:
                    assert_attention_close(got.cpu().numpy().reshape(-1), want, "head-sharded decode vs the oracle")
                except AssertionError:
                    ok_oracle = False
        q_out.put((rank, ok_bits, ok_oracle))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_head_sharded_decode_all_gathers_to_the_single_gpu_result():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q_out)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(q_out.get(timeout=300) for _ in procs)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert results == [(0, True, True), (1, True, True)]
