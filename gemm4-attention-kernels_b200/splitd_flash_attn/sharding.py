"""Data-parallel sharding of an attention layer over the GPUs of one node.

Attention is independent per (batch, KV-head group) and per packed sequence, and the GQA reduction of
dK/dV stays inside one KV-head group (src/fmha_dkdv_sm90_d512.py:895-936 of the reference), so shards
never exchange data: there is no collective on the hot path. torch.distributed is used only to agree on
timings and to gather per-shard check results.
"""

from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

import torch
import torch.distributed as dist


def layer_shards(batch: int, heads_kv: int) -> List[Tuple[int, int]]:
    """All (batch index, KV head) shards of a (B, S, Hq, D) layer, in a fixed order."""
    return [(b, h) for b in range(batch) for h in range(heads_kv)]


def shards_of_rank(n_shards: int, rank: int, world: int) -> List[int]:
    """Round-robin assignment; every shard goes to exactly one rank."""
    return list(range(rank, n_shards, world))


def shard_views(q, k, v, shard: Tuple[int, int], heads_q: int, heads_kv: int):
    """Strided views (no copy) of one shard: q[b, :, g*G:(g+1)*G], k/v[b, :, g:g+1]."""
    b, g = shard
    group = heads_q // heads_kv
    return q[b : b + 1, :, g * group : (g + 1) * group], k[b : b + 1, :, g : g + 1], v[b : b + 1, :, g : g + 1]


def max_over_ranks(value: float, device) -> float:
    """Largest value over all ranks (used for the step time: the slowest rank defines the step)."""
    t = torch.tensor([value], dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def gather_shard_results(local: Dict[int, float], n_shards: int, device) -> List[float]:
    """Every rank contributes the results of its own shards; returns the full per-shard list."""
    t = torch.full((n_shards,), float("-inf"), dtype=torch.float64, device=device)
    for i, val in local.items():
        t[i] = val
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()
