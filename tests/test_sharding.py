"""Sequence sharding, the kv-head partition of a prefill chunk with its all-gather and token-major placement, and the
max-over-ranks timing reduction, on 2 gloo ranks (CPU)."""
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


def _slab_value(tok, col):
    """A value that names its place in o[T][Hq * 128]."""
    return (tok * 2048 + col).to(torch.float32)


def test_prefill_partition_tiles_heads_and_tokens():
    Hq, Hkv, T = 16, 4, 2048
    for world in (1, 2, 4, 8):
        cover = torch.zeros(T, Hq, dtype=torch.int32)
        for r in range(world):
            sh = shard.prefill_partition(Hq, Hkv, T, world, r)
            assert sh.kv_shards * sh.tok_shards == world and sh.n_q_heads == sh.n_kv_heads * (Hq // Hkv)
            assert sh.q_head0 == sh.kv_head0 * (Hq // Hkv)
            cover[sh.token0:sh.token0 + sh.n_tokens, sh.q_head0:sh.q_head0 + sh.n_q_heads] += 1
        assert bool((cover == 1).all()), f"{world} ranks do not tile the chunk exactly once"
    sh = shard.prefill_partition(Hq, Hkv, T, 8, 5)       # kv head 2, second half of the chunk
    assert (sh.kv_head0, sh.n_kv_heads, sh.token0, sh.n_tokens) == (2, 1, 1024, 1024)
    with pytest.raises(ValueError):
        shard.prefill_partition(Hq, Hkv, T, 3, 0)
    with pytest.raises(ValueError):
        shard.prefill_partition(Hq, Hkv, 2047, 8, 0)


def test_place_heads_is_the_inverse_of_the_partition():
    Hq, Hkv, T = 16, 4, 64
    tok = torch.arange(T)[:, None]
    col = torch.arange(Hq * 128)[None, :]
    want = _slab_value(tok, col)
    for world in (2, 4, 8):
        slabs = []
        for r in range(world):
            sh = shard.prefill_partition(Hq, Hkv, T, world, r)
            slabs.append(want[sh.token0:sh.token0 + sh.n_tokens, sh.q_head0 * 128:(sh.q_head0 + sh.n_q_heads) * 128])
        gathered = torch.stack(slabs).contiguous()
        sh = shard.prefill_partition(Hq, Hkv, T, world, 0)
        got = shard.place_heads(gathered, torch.zeros(T, Hq * 128), sh.kv_shards, sh.tok_shards)
        assert torch.equal(got, want)


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    first, count = shard.shard_sequences(64, world, rank)
    mine = torch.zeros(64)
    mine[first:first + count] = 1.0
    dist.all_reduce(mine)                                   # every sequence owned exactly once across ranks
    slowest = shard.max_over_ranks(10.0 + rank)             # step time = the slowest rank's
    # the head-sharded prefill's combine: every rank contributes the slab of its kv heads, one all-gather, token-major placement
    Hq, Hkv, T = 16, 4, 32
    sh = shard.prefill_partition(Hq, Hkv, T, world, rank)
    tok = torch.arange(sh.token0, sh.token0 + sh.n_tokens)[:, None]
    col = torch.arange(sh.q_head0 * 128, (sh.q_head0 + sh.n_q_heads) * 128)[None, :]
    local = _slab_value(tok, col).contiguous()
    gathered = torch.zeros(world, sh.n_tokens, sh.n_q_heads * 128)
    shard.all_gather_rows(gathered, local)
    o = shard.place_heads(gathered, torch.zeros(T, Hq * 128), sh.kv_shards, sh.tok_shards)
    placed = bool(torch.equal(o, _slab_value(torch.arange(T)[:, None], torch.arange(Hq * 128)[None, :])))
    dist.barrier()
    if rank == 0:
        out.put((mine.tolist(), slowest, placed))
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
    owned, slowest, placed = out.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert owned == [1.0] * 64
    assert slowest == 11.0
    assert placed, "all-gather + placement did not rebuild the token-major output"
