"""How the attention work shards across the GPUs of one box.

Every (batch, KV-head group) of a prefill call and every sequence of a decode
call is independent, so there is no exchange step: each rank runs the single-GPU
kernel on its shard and no collective touches the data path.  Only a caller that
wants the whole output on every rank pays for an all-gather (`gather_output`),
the analogue of lean_torch_dist_all_gather_into_tensor
(cc/src/tyr_distributed.cpp:493-538), which chunks along dim 0.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence, Tuple

import torch


@dataclass(frozen=True)
class PrefillShard:
    batch: Tuple[int, int]      # [begin, end) over the batch
    kv_heads: Tuple[int, int]   # [begin, end) over KV heads (query heads follow: h*g..)
    axis: str                   # "heads" | "batch" | "batch*heads"


def _even(n: int, parts: int, i: int) -> Tuple[int, int]:
    base, rem = divmod(n, parts)
    lo = i * base + min(i, rem)
    return lo, lo + base + (1 if i < rem else 0)


def prefill_shard(batch: int, n_kv_head: int, world: int, rank: int) -> PrefillShard:
    """Split by KV-head group when the head count divides (one group per GPU at
    world = n_kv_head), else by batch, else on a (batch x heads) grid."""
    if not 0 <= rank < world:
        raise ValueError("rank out of range")
    if world == 1:
        return PrefillShard((0, batch), (0, n_kv_head), "heads")
    if n_kv_head % world == 0:
        return PrefillShard((0, batch), _even(n_kv_head, world, rank), "heads")
    if batch % world == 0:
        return PrefillShard(_even(batch, world, rank), (0, n_kv_head), "batch")
    for wb in range(min(world, batch), 0, -1):      # largest batch factor that fits
        if world % wb == 0 and batch % wb == 0 and n_kv_head % (world // wb) == 0:
            wh = world // wb
            return PrefillShard(_even(batch, wb, rank // wh), _even(n_kv_head, wh, rank % wh),
                                "batch*heads")
    # uneven: contiguous runs of (batch, head) units, cut on the batch axis only
    return PrefillShard(_even(batch, world, rank), (0, n_kv_head), "batch")


def slice_prefill(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, shard: PrefillShard):
    """Views of this rank's part of q [B,Hq,S,D] and k, v [B,Hkv,S,D]."""
    g = q.shape[1] // k.shape[1]
    (b0, b1), (h0, h1) = shard.batch, shard.kv_heads
    return (q[b0:b1, h0 * g:h1 * g], k[b0:b1, h0:h1], v[b0:b1, h0:h1])


def lpt_partition(lengths: Sequence[int], world: int) -> List[List[int]]:
    """Greedy length-balanced split of decode sequences: longest first, each to
    the least-loaded rank.  Returns the sequence indices of every rank."""
    if world <= 0:
        raise ValueError("world must be positive")
    loads = [0] * world
    out: List[List[int]] = [[] for _ in range(world)]
    for i in sorted(range(len(lengths)), key=lambda i: (-lengths[i], i)):
        r = min(range(world), key=lambda r: (loads[r], r))
        out[r].append(i)
        loads[r] += lengths[i]
    return out


def gather_output(o_shard: torch.Tensor, shard_axis: str, group=None) -> torch.Tensor:
    """Replicate the output on every rank (only when the caller asks for it).

    One all_gather_into_tensor of the equal-sized shards into a [world, ...]
    staging buffer in local memory, then a local permute to [B, Hq, S, D].
    """
    import torch.distributed as dist
    world = dist.get_world_size(group)
    o_shard = o_shard.contiguous()
    flat = torch.empty((world * o_shard.shape[0],) + tuple(o_shard.shape[1:]), dtype=o_shard.dtype,
                       device=o_shard.device)
    dist.all_gather_into_tensor(flat, o_shard, group=group)   # rank r's shard lands in chunk r of dim 0
    stage = flat.view((world,) + tuple(o_shard.shape))
    if shard_axis == "batch":
        return stage.reshape((-1,) + tuple(o_shard.shape[1:]))
    if shard_axis == "heads":
        # [world, B, h, S, D] -> [B, world*h, S, D]
        return stage.permute(1, 0, 2, 3, 4).reshape(o_shard.shape[0], -1, *o_shard.shape[2:])
    raise ValueError("gather_output handles the 'batch' and 'heads' splits")
