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


_TILE_KEYS = ("bm_qkv", "bn_qkv", "bm_proj", "bn_proj", "split_proj", "bm_fc1", "bn_fc1", "bm_fc2", "bn_fc2", "split_fc2")


def encoder_with_common_tiling(build, rank: int, world: int, group=None):
    """One encoder per rank, all with the SAME tilings: `build(tuning)` makes a `bert.BertEncoder` for this rank's shard.

    Rank 0 lets the library time the candidate tilings on its device (tuning autotune = 1) and broadcasts what it
    chose (tile heights, widths and split-K depths of the four GEMM stages); the other ranks build their plans with
    those values.  Timing is noisy enough that two ranks would otherwise now and then settle on different split-K
    depths, and with them on different summation orders: the ranks' outputs for the same sequence would then differ
    in the last bit, and their step times by a few per cent."""
    if world == 1:
        return build({"autotune": 1})
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    choice = torch.zeros(len(_TILE_KEYS), dtype=torch.int64, device=dev)
    enc = None
    if rank == 0:
        enc = build({"autotune": 1})
        q, p, f1, f2 = (enc.stage_info(i) for i in (0, 2, 4, 5))      # QKV, proj, FC1, FC2 of the first layer
        choice = torch.tensor([q["bm"], q["bn"], p["bm"], p["bn"], p["splitk"], f1["bm"], f1["bn"], f2["bm"], f2["bn"],
                               f2["splitk"]], dtype=torch.int64, device=dev)
    dist.broadcast(choice, 0, group=group)
    if rank != 0:
        enc = build(dict(zip(_TILE_KEYS, (int(v) for v in choice.tolist()))))
    return enc


class ShardedHostPipeline:
    """One rank's end-to-end step of the sharded encoder with HOST buffers on both sides:

        pinned shard -> device  |  encoder on the shard  |  all-gather over NVLink  |  this rank's slice of the
        gathered batch -> host

    Consecutive steps are pipelined over a copy-in stream, the caller's current stream (encoder + gather) and a
    copy-out stream, with two sets of device buffers, so the copies of one step run under the kernel of its
    neighbours -- what souffle_bert_forward_host_async does inside the library for the single-GPU case.  Every rank
    reads back its own 1/world of the gathered result, so the whole batch reaches host memory once per step, spread
    over the rank processes like the inputs.

    `forward(x_dev, lens_dev, y_dev)` is the rank's encoder (BertEncoder.forward).  With CPU tensors (gloo tests) the
    same steps run synchronously without streams.
    """

    def __init__(self, forward, x_like: torch.Tensor, lens_like: Optional[torch.Tensor], rank: int, world: int,
                 group: Optional[dist.ProcessGroup] = None):
        self.forward, self.rank, self.world, self.group = forward, rank, world, group
        self.per = x_like.shape[0]
        self.cuda = x_like.is_cuda
        n = 2 if self.cuda else 1
        self.x = [torch.empty_like(x_like) for _ in range(n)]
        self.l = [torch.empty_like(lens_like) if lens_like is not None else None for _ in range(n)]
        self.y = [torch.empty_like(x_like) for _ in range(n)]
        full_shape = (self.per * world,) + tuple(x_like.shape[1:])
        self.full = [torch.empty(full_shape, dtype=x_like.dtype, device=x_like.device) for _ in range(n)]
        self.calls = 0
        if self.cuda:
            self.s_in, self.s_out = torch.cuda.Stream(), torch.cuda.Stream()
            self.ev_k, self.ev_out = [None, None], [None, None]

    def step(self, x_host: torch.Tensor, lens_host: Optional[torch.Tensor], out_host: torch.Tensor) -> torch.Tensor:
        """Queues one step; `out_host` ([per, ...]) is complete after drain() (or once a later step that reuses the
        same buffer set has been queued and the current stream has caught up).  Returns the device tensor that will
        hold the gathered batch of this step."""
        b = self.calls & 1 if self.cuda else 0
        self.calls += 1
        lo, hi = self.rank * self.per, (self.rank + 1) * self.per
        if not self.cuda:
            self.x[b].copy_(x_host)
            if lens_host is not None:
                self.l[b].copy_(lens_host)
            self.forward(self.x[b], self.l[b], self.y[b])
            gather_outputs(self.y[b], self.full[b], self.group) if self.world > 1 else self.full[b].copy_(self.y[b])
            out_host.copy_(self.full[b][lo:hi])
            return self.full[b]
        cur = torch.cuda.current_stream()
        with torch.cuda.stream(self.s_in):
            if self.ev_k[b] is not None:
                self.s_in.wait_event(self.ev_k[b])             # the encoder of the step before last has read x[b]
            self.x[b].copy_(x_host, non_blocking=True)
            if lens_host is not None:
                self.l[b].copy_(lens_host, non_blocking=True)
            ev_in = self.s_in.record_event()
        cur.wait_event(ev_in)
        if self.ev_out[b] is not None:
            cur.wait_event(self.ev_out[b])                     # full[b] has been copied out
        self.forward(self.x[b], self.l[b], self.y[b])
        if self.world > 1:
            gather_outputs(self.y[b], self.full[b], self.group)
        else:
            self.full[b].copy_(self.y[b])
        self.ev_k[b] = cur.record_event()
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.ev_k[b])
            out_host.copy_(self.full[b][lo:hi], non_blocking=True)
            self.ev_out[b] = self.s_out.record_event()
        return self.full[b]

    def drain(self) -> None:
        """Makes the current stream wait for every copy-out queued so far."""
        if self.cuda:
            for ev in self.ev_out:
                if ev is not None:
                    torch.cuda.current_stream().wait_event(ev)
