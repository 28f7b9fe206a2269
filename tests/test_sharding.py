"""Sequence sharding and the max-over-ranks timing reduction, on 2 gloo ranks (CPU)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from embla_metal_b200 import shard


def test_shards_cover_every_sequence_once():
    for total in (64, 7, 1, 0):
        for world in (1, 2, 3, 4, 8):
            seen = []
            for r in range(world):
                first, count = shard.shard_sequences(total, world, r)
                seen += list(range(first, first + count))
            assert seen == list(range(total))
            counts = [shard.shard_sequences(total, world, r)[1] for r in range(world)]
            assert max(counts) - min(counts) <= 1
    with pytest.raises(ValueError):
        shard.shard_sequences(4, 2, 2)


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    first, count = shard.shard_sequences(64, world, rank)
    mine = torch.zeros(64)
    mine[first:first + count] = 1.0
    dist.all_reduce(mine)                                   # every sequence owned exactly once across ranks
    slowest = shard.max_over_ranks(10.0 + rank)             # step time = the slowest rank's
    dist.barrier()
    if rank == 0:
        out.put((mine.tolist(), slowest))
    dist.destroy_process_group()


def test_two_gloo_ranks():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    owned, slowest = out.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert owned == [1.0] * 64
    assert slowest == 11.0
