"""Batch sharding of the encoder across GPUs: one process per GPU, weights replicated,
sequences split evenly, one all-gather of the final activations.

The reference has no multi-GPU code at all (device 0 is hard-wired in
cpp/souffle_utils/torch_utils.h:5-29); sequences never interact inside an encoder layer, so the
path partitions by sequence with no data-path collective, and the only exchange is the output
gather.  Works with the NCCL backend on GPUs and with gloo on CPU (used by the tests).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist


def shard_range(batch: int, rank: int, world: int) -> Tuple[int, int]:
    """[begin, end) of the sequences rank `rank` owns.  The batch must divide evenly so every
    rank runs the same plan shape (required for one all-gather into a dense tensor)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world {rank}/{world}")
    if batch % world:
        raise ValueError(f"batch {batch} is not divisible by world size {world}")
    per = batch // world
    return rank * per, (rank + 1) * per


def shard_batch(x: torch.Tensor, lens: Optional[torch.Tensor], rank: int, world: int):
    """Slices [B, S, H] activations (and [B] lengths) to this rank's sequences."""
    b0, b1 = shard_range(x.shape[0], rank, world)
    return x[b0:b1].contiguous(), (lens[b0:b1].contiguous() if lens is not None else None)


def gather_outputs(local: torch.Tensor, out: Optional[torch.Tensor] = None,
                   group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """All-gathers [B/world, S, H] shards into [B, S, H] on every rank (rank order = batch order)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return local
    if out is None:
        out = torch.empty((local.shape[0] * world,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(out, local.contiguous(), group=group)
    return out
