"""Partition of a batch of independent sequences over ranks, and the max-over-ranks time reduction.

Batched decode shards by sequence with no data-path collective; the only communication is the
timing plumbing (a barrier and a MAX all-reduce), which works on any torch.distributed backend
(nccl on GPUs, gloo in the CPU tests).
"""
import torch


def shard_sequences(total, world, rank):
    """Contiguous, balanced share of `total` sequences for `rank` of `world`: (first, count)."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} of {world}")
    base, extra = divmod(total, world)
    count = base + (1 if rank < extra else 0)
    first = rank * base + min(rank, extra)
    return first, count


def max_over_ranks(value, device="cpu", group=None):
    """MAX of a python float over the ranks of the default (or given) process group."""
    import torch.distributed as dist
    t = torch.tensor([float(value)], device=device)
    if dist.is_available() and dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
