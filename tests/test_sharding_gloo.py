"""Multi-process host logic on CPU (gloo, world_size 2): sequence placement and the
all-gather of head-sharded outputs, with the oracle standing in for the kernels."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from combsengine_b200.sharding import admit_to_rank, all_gather_heads, kv_head_range, partition_sequences


def test_partition_is_balanced_and_complete():
    rng = np.random.default_rng(5)
    lens = np.round(np.exp(rng.uniform(np.log(128), np.log(32768), 512))).astype(int) + 1024
    parts = partition_sequences(lens, 8)
    assert sorted(i for p in parts for i in p) == list(range(512))
    loads = [sum(-(-int(lens[i]) // 16) for i in p) for p in parts]
    assert max(loads) - min(loads) <= max(-(-int(x) // 16) for x in lens)  # LPT bound
    assert max(loads) / (sum(loads) / 8) < 1.02
    assert partition_sequences([5, 5, 5], 2) == [[0, 2], [1]]
    assert admit_to_rank([10, 30, 30, 5]) == 1


def _worker(rank, world, port, q_out):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import OracleArena
        n_q, n_kv, d, L = 8, 4, 64, 70
        rng = np.random.default_rng(99)  # the same inputs on every rank
        q = rng.standard_normal((n_q, L, d)).astype(np.float16)
        k = rng.standard_normal((n_kv, L, d)).astype(np.float16)
        v = rng.standard_normal((n_kv, L, d)).astype(np.float16)
        heads = kv_head_range(n_kv, rank, world)
        rep = n_q // n_kv
        qh = q[heads.start * rep: heads.stop * rep]
        arena = OracleArena(1, len(heads), d, 256, dtype="f16")
        out_shard = arena.new_seq().attention(0, qh, k[heads.start:heads.stop], v[heads.start:heads.stop], 0, d ** -0.5)
        # [tokens, heads, d] as the gather expects
        shard = torch.from_numpy(np.ascontiguousarray(out_shard.transpose(1, 0, 2)))
        full = all_gather_heads(shard).numpy().transpose(1, 0, 2)
        ref_arena = OracleArena(1, n_kv, d, 256, dtype="f16")
        ref = ref_arena.new_seq().attention(0, q, k, v, 0, d ** -0.5)
        q_out.put((rank, bool(np.array_equal(full.view(np.uint16), ref.view(np.uint16)))))
    finally:
        dist.destroy_process_group()


def test_head_sharded_outputs_all_gather_to_the_unsharded_result():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q_out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q_out.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(0, True), (1, True)]
