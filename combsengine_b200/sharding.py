"""Placement of sequences and heads on several GPUs (one process per GPU).

The path shards by sequence: every sequence's pages, block table and attention are
independent (the reference is literally one cache object per sequence,
``kv.rs:477-495``), so ranks exchange nothing inside the path.  For models whose KV
heads are split across GPUs instead, each rank attends its own KV-head group and the
head-sharded outputs are put back together with one all-gather per layer.
"""
from __future__ import annotations

from typing import List, Sequence

import torch
import torch.distributed as dist


def pages_of(length: int, page_size: int = 16) -> int:
    return -(-int(length) // page_size)


def partition_sequences(lengths: Sequence[int], world: int, page_size: int = 16) -> List[List[int]]:
    """Longest-processing-time-first assignment of sequences to ranks by page count.

    Decode cost is proportional to the pages a sequence reads, so this balances the bytes
    each GPU streams per step.  Returns, per rank, the indices of its sequences in
    ascending order (deterministic: ties go to the lower rank).
    """
    order = sorted(range(len(lengths)), key=lambda i: (-pages_of(lengths[i], page_size), i))
    load = [0] * world
    out: List[List[int]] = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda j: (load[j], j))
        out[r].append(i)
        load[r] += pages_of(lengths[i], page_size)
    return [sorted(x) for x in out]


def admit_to_rank(free_pages: Sequence[int]) -> int:
    """A newly admitted sequence goes to the rank with the most free pages."""
    return max(range(len(free_pages)), key=lambda j: (free_pages[j], -j))


def kv_head_range(n_kv_heads: int, rank: int, world: int) -> range:
    """KV heads owned by `rank` when heads are sharded (contiguous groups)."""
    if n_kv_heads % world:
        raise ValueError("n_kv_heads must be divisible by the number of ranks")
    per = n_kv_heads // world
    return range(rank * per, (rank + 1) * per)


def all_gather_heads(out_shard: torch.Tensor, group=None) -> torch.Tensor:
    """Head-sharded attention outputs ``[tokens, n_q / world, d]`` -> ``[tokens, n_q, d]``.

    One all-gather per layer (NCCL over NVLink on GPUs, gloo in the CPU tests); rank r's
    q heads are the r-th contiguous block, matching ``kv_head_range``.
    """
    world = dist.get_world_size(group)
    parts = [torch.empty_like(out_shard) for _ in range(world)]
    dist.all_gather(parts, out_shard.contiguous(), group=group)
    return torch.cat(parts, dim=1)
