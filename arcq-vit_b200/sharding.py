"""Batch sharding of whole-model inference over the GPUs of one box.

Images are independent and the packed model (<= 60 MB for DeiT-B) is replicated, so rank r of W
takes a contiguous slice of the global batch and the only exchange is one all-gather of logits
per global batch.  No collective runs inside a layer.  Works on NCCL (GPU) and gloo (CPU tests).
The reference has no counterpart: its only parallelism is DDP in training
(methods/fair_qat_framework/fair_qat/train_imagenet_qat.py:35-45, :664-683).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist


def shard_bounds(global_batch: int, world_size: int, rank: int) -> Tuple[int, int]:
    """[start, end) of rank's slice: the first ``global_batch % world_size`` ranks get one more."""
    if world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError(f"bad rank {rank} of {world_size}")
    base, extra = divmod(global_batch, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def gather_logits(local_logits: torch.Tensor, global_batch: int, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """All ranks receive [global_batch, classes] in global image order.  Slices may be uneven
    (by at most one row); they are padded to the largest for the collective and trimmed after."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return local_logits
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    s, e = shard_bounds(global_batch, world, rank)
    if local_logits.shape[0] != e - s:
        raise ValueError(f"rank {rank} holds {local_logits.shape[0]} rows, its shard has {e - s}")
    width = -(-global_batch // world)
    buf = local_logits.new_zeros((width,) + tuple(local_logits.shape[1:]))
    buf[: e - s] = local_logits
    out = local_logits.new_empty((world * width,) + tuple(local_logits.shape[1:]))
    dist.all_gather_into_tensor(out, buf.contiguous(), group=group)
    parts = []
    for r in range(world):
        rs, re = shard_bounds(global_batch, world, r)
        parts.append(out[r * width: r * width + (re - rs)])
    return torch.cat(parts, dim=0)
