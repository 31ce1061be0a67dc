"""KV-head sharding of the decode path over the GPUs of one node.

Each (sequence, kv head) pair is independent on this path (the reference maps query head h to kv head
h // group, src/kernels/src/pagedattention.cu:147-150), so rank r of N owns kv heads
[r * KVH / N, (r + 1) * KVH / N), the matching contiguous range of query heads, their ALiBi slopes and a
private cache slice.  Block tables, context lengths and slot mappings are replicated.  Nothing is
exchanged on the attention path; the only collective offered here is the optional all-gather of the
per-rank outputs, for callers that want the full [seqs, heads, d] tensor on every rank.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch


def head_ranges(rank: int, world: int, num_heads: int, num_kv_heads: int) -> Tuple[int, int, int, int]:
    """(kv_lo, kv_hi, q_lo, q_hi) owned by ``rank``."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    if num_kv_heads % world != 0:
        raise ValueError(f"{num_kv_heads} kv heads do not split evenly over {world} ranks")
    if num_heads % num_kv_heads != 0:
        raise ValueError(f"{num_heads} query heads are not a multiple of {num_kv_heads} kv heads")
    group = num_heads // num_kv_heads
    per = num_kv_heads // world
    return rank * per, (rank + 1) * per, rank * per * group, (rank + 1) * per * group


def shard_query(q: torch.Tensor, rank: int, world: int, num_kv_heads: int) -> torch.Tensor:
    """This rank's query heads: a view of q, row stride unchanged (the kernels take a strided q)."""
    _, _, lo, hi = head_ranges(rank, world, q.shape[1], num_kv_heads)
    return q[:, lo:hi]


def shard_cache(cache: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """This rank's private slice of a key or value cache ([num_blocks, kv_heads, ...]), made contiguous."""
    kvh = cache.shape[1]
    if kvh % world != 0:
        raise ValueError(f"{kvh} kv heads do not split evenly over {world} ranks")
    per = kvh // world
    return cache[:, rank * per:(rank + 1) * per].contiguous()


def shard_rows(x: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """This rank's heads of new key / value rows ([tokens, kv_heads, d]): a strided view."""
    per = x.shape[1] // world
    return x[:, rank * per:(rank + 1) * per]


def shard_slopes(slopes: Optional[torch.Tensor], rank: int, world: int, num_kv_heads: int) -> Optional[torch.Tensor]:
    if slopes is None:
        return None
    _, _, lo, hi = head_ranges(rank, world, slopes.shape[0], num_kv_heads)
    return slopes[lo:hi].contiguous()


def gather_heads(out_local: torch.Tensor, group=None) -> torch.Tensor:
    """All-gathers per-rank outputs [seqs, heads / N, d] into [seqs, heads, d] on every rank."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    if world == 1:
        return out_local
    ns, nh, hs = out_local.shape
    buf = torch.empty((world * ns, nh, hs), dtype=out_local.dtype, device=out_local.device)   # rank-major
    dist.all_gather_into_tensor(buf, out_local.contiguous(), group=group)
    return buf.view(world, ns, nh, hs).permute(1, 0, 2, 3).reshape(ns, world * nh, hs)


def max_over_ranks(value: float, device, group=None) -> float:
    """The slowest rank's figure: what a multi-GPU timing must report."""
    import torch.distributed as dist
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t[0])
