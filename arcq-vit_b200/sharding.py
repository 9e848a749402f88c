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


class LogitsGatherer:
    """All-gather of even shards off the critical path.

    ``submit(local)`` copies this rank's logits (a small tensor: [B/W, classes]) into one of two staging rows on
    the caller's stream and issues ``all_gather_into_tensor`` from there straight into a preallocated
    [B, classes] buffer on a side stream behind an event, so the next forward runs while the collective (a few
    tens of microseconds, latency-bound) is in flight.  ``result()`` waits for the newest gather and returns its
    buffer, rows in global image order.  On CPU tensors (gloo tests) everything runs inline.  Uneven shards go
    through ``gather_logits``.
    """

    def __init__(self, global_batch: int, classes: int, dtype: torch.dtype, device: torch.device,
                 group: Optional[dist.ProcessGroup] = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if global_batch % self.world != 0:
            raise ValueError(f"global batch {global_batch} does not split evenly over {self.world} ranks")
        self.local_rows = global_batch // self.world
        self.cuda = device.type == "cuda"
        self.stage = [torch.empty((self.local_rows, classes), dtype=dtype, device=device) for _ in range(2)]
        self.out = [torch.empty((global_batch, classes), dtype=dtype, device=device) for _ in range(2)]
        self.side = torch.cuda.Stream(device=device) if self.cuda else None
        self.ready = [torch.cuda.Event() for _ in range(2)] if self.cuda else None
        self.done = [torch.cuda.Event() for _ in range(2)] if self.cuda else None
        self.n = 0

    def submit(self, local_logits: torch.Tensor) -> None:
        if tuple(local_logits.shape) != tuple(self.stage[0].shape):
            raise ValueError(f"rank {self.rank} holds {tuple(local_logits.shape)}, its shard is {tuple(self.stage[0].shape)}")
        s = self.n & 1
        self.n += 1
        if self.world == 1:
            self.out[s].copy_(local_logits)
            return
        if not self.cuda:
            self.stage[s].copy_(local_logits)
            dist.all_gather_into_tensor(self.out[s], self.stage[s], group=self.group)
            return
        cur = torch.cuda.current_stream()
        if self.n > 2:
            cur.wait_event(self.done[s])            # the gather that last read this staging row has finished
        self.stage[s].copy_(local_logits, non_blocking=True)
        self.ready[s].record(cur)
        with torch.cuda.stream(self.side):
            self.side.wait_event(self.ready[s])
            dist.all_gather_into_tensor(self.out[s], self.stage[s], group=self.group)
            self.done[s].record(self.side)

    def result(self) -> torch.Tensor:
        """The newest gathered [global_batch, classes] tensor (the caller's stream waits for its gather)."""
        if self.n == 0:
            raise RuntimeError("nothing was submitted")
        s = (self.n - 1) & 1
        if self.cuda and self.world > 1:
            torch.cuda.current_stream().wait_event(self.done[s])
        return self.out[s]
