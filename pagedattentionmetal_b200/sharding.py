"""KV-head sharding across the GPUs of one node (host-side helpers).

GPU r of N owns KV heads [r*KVH/N, (r+1)*KVH/N) and the query heads that map to
them; attention for a query head reads only its KV head (kernels.metal:1439,
kv_head = head / (heads / kv_heads)), so no collective runs on the attention
path.  Every rank takes the same allocator decisions (same calls in the same
order), hence identical block tables.  `gather_heads` is the optional
all-gather of per-head outputs for callers that need the full tensor.
"""
from __future__ import annotations

from typing import Tuple


def head_range(rank: int, world: int, num_heads: int, num_kv_heads: int) -> Tuple[int, int, int, int]:
    """(q_lo, q_hi, kv_lo, kv_hi) owned by `rank`."""
    if num_kv_heads % world or num_heads % num_kv_heads:
        raise ValueError("KV heads must divide over the ranks and query heads over the KV heads")
    kv_per = num_kv_heads // world
    group = num_heads // num_kv_heads
    return rank * kv_per * group, (rank + 1) * kv_per * group, rank * kv_per, (rank + 1) * kv_per


def shard_heads(x, rank: int, world: int, axis: int):
    """Slice of `x` (numpy array or torch tensor) along a head axis for `rank`."""
    n = x.shape[axis]
    if n % world:
        raise ValueError("head axis does not divide over the ranks")
    per = n // world
    index = [slice(None)] * x.ndim
    index[axis] = slice(rank * per, (rank + 1) * per)
    return x[tuple(index)]


def gather_heads(local_out, group=None):
    """All-gather `[rows][local_heads][dim]` torch tensors of every rank into
    `[rows][heads][dim]` (torch.distributed; NCCL on GPUs, gloo on CPU)."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    parts = [torch.empty_like(local_out) for _ in range(world)]
    dist.all_gather(parts, local_out.contiguous(), group=group)
    return torch.cat(parts, dim=1)
