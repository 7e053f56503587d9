"""Batch sharding + output gather, exercised with two gloo ranks on CPU."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from souffle_models_b200 import sharding


def test_shard_range():
    assert sharding.shard_range(64, 0, 1) == (0, 64)
    assert [sharding.shard_range(64, r, 8) for r in range(8)] == [(8 * r, 8 * r + 8) for r in range(8)]
    with pytest.raises(ValueError):
        sharding.shard_range(10, 0, 4)
    with pytest.raises(ValueError):
        sharding.shard_range(8, 2, 2)


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(7)
        x = torch.randn(8, 4, 16, generator=g)
        lens = torch.arange(8, dtype=torch.int32)
        xs, ls = sharding.shard_batch(x, lens, rank, world)
        assert xs.shape[0] == 8 // world and torch.equal(ls, lens[rank * 4:(rank + 1) * 4])
        y_local = xs * 2 + 1                      # stands in for the per-rank encoder
        full = sharding.gather_outputs(y_local)
        ok = bool(torch.equal(full, x * 2 + 1))
        # the host-buffer pipeline (synchronous on CPU): shard in, "encoder", gather, this rank's slice back out
        pipe = sharding.ShardedHostPipeline(lambda xd, ld, yd: yd.copy_(xd * 2 + 1), xs, ls, rank, world)
        out = torch.empty_like(xs)
        for _ in range(3):
            gathered = pipe.step(xs, ls, out)
        pipe.drain()
        ok = ok and bool(torch.equal(gathered, x * 2 + 1)) and bool(torch.equal(out, xs * 2 + 1))
        # common tilings: rank 0 "times" them, the other rank is built from its choice

        class FakeEncoder:
            def __init__(self, tuning):
                self.tuning = tuning

            def stage_info(self, i):
                return {0: dict(bm=128, bn=256, splitk=1), 2: dict(bm=256, bn=192, splitk=1), 4: dict(bm=128, bn=256, splitk=1),
                        5: dict(bm=256, bn=192, splitk=2)}[i]

        enc = sharding.encoder_with_common_tiling(FakeEncoder, rank, world)
        want = dict(bm_qkv=128, bn_qkv=256, bm_proj=256, bn_proj=192, split_proj=1, bm_fc1=128, bn_fc1=256, bm_fc2=256,
                    bn_fc2=192, split_fc2=2)
        ok = ok and enc.tuning == ({"autotune": 1} if rank == 0 else want)
        ret[rank] = ok
    finally:
        dist.destroy_process_group()


def test_two_rank_gather_reassembles_the_batch():
    world = 2
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_worker, args=(world, 29531 + os.getpid() % 200, ret), nprocs=world, join=True)
        assert ret[0] and ret[1]


def test_single_rank_gather_is_identity():
    t = torch.ones(2, 3)
    assert sharding.gather_outputs(t) is t
