"""How the attention path spreads over the GPUs of one box.

* Batched decode shards by sequence: sequences are independent, every GPU holds the KV state of its own,
  and nothing crosses GPUs on the data path (`shard_sequences`).
* A long prefill chunk of a full layer shards by kv head: a GPU holds the cache pages of its kv heads
  only and computes their query heads (`prefill_partition`); with more GPUs than kv heads the chunk's
  tokens are cut as well. Every GPU ends up with the token-major `o[T][n_q_heads * 128]` that the
  o-projection after attention reads (the reference's single GPU writes that layout directly,
  Sources/EmblaMetal/Prefill.swift:343-344, 378-407). `HeadShardedPrefill` is that path as one object,
  two ways: the kernel's epilogue stores every output row into all GPUs' outputs itself, over NVLink into
  symmetric memory, followed by one barrier across the GPUs (`fused=True`: compute and all-gather are one
  kernel); or the kernel writes a local slab, one NCCL all-gather (gloo in the CPU tests) collects the slabs
  and a strided copy places them.

The only other communication is the timing plumbing (`max_over_ranks`). No kernel of this library READS
another GPU's memory; the fused path writes into it with plain stores.
"""
from collections import namedtuple

import torch

PrefillShard = namedtuple("PrefillShard", "kv_shards tok_shards kv_part tok_part kv_head0 n_kv_heads q_head0 n_q_heads "
                                          "token0 n_tokens")


def shard_sequences(total, world, rank):
    """Contiguous, balanced share of `total` sequences for `rank` of `world`: (first, count)."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} of {world}")
    base, extra = divmod(total, world)
    count = base + (1 if rank < extra else 0)
    first = rank * base + min(rank, extra)
    return first, count


def prefill_partition(n_q_heads, n_kv_heads, n_tokens, world, rank):
    """Which kv heads, query heads and tokens of a prefill chunk `rank` of `world` computes.

    Ranks split the kv heads first (rank // tok_shards picks the group of kv heads); once there are more
    ranks than kv heads, the ranks of one kv head split the chunk's tokens into contiguous runs
    (rank % tok_shards). With 4 kv heads: 2 GPUs take 2 kv heads each, 4 take one each, 8 take one kv
    head and one half of the chunk each (the kv head's pages are then held by both)."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} of {world}")
    kv_shards = min(world, n_kv_heads)
    if n_kv_heads % kv_shards or world % kv_shards:
        raise ValueError(f"{world} ranks do not divide {n_kv_heads} kv heads evenly")
    tok_shards = world // kv_shards
    if n_tokens % tok_shards:
        raise ValueError(f"{n_tokens} tokens do not divide over {tok_shards} ranks a kv head")
    g = n_q_heads // n_kv_heads
    kv_part, tok_part = rank // tok_shards, rank % tok_shards
    hkv = n_kv_heads // kv_shards
    t = n_tokens // tok_shards
    return PrefillShard(kv_shards, tok_shards, kv_part, tok_part, kv_part * hkv, hkv, kv_part * hkv * g, hkv * g,
                        tok_part * t, t)


def place_heads(gathered, o_full, kv_shards, tok_shards):
    """gathered [world][T_l][hq_l * 128] as an all-gather leaves it (rank-major) -> o_full [T][Hq * 128], token-major:
    rank kv_part * tok_shards + tok_part holds tokens tok_part * T_l .. and heads kv_part * hq_l .. One strided copy."""
    world, t_l, w_l = gathered.shape
    if world != kv_shards * tok_shards or tuple(o_full.shape) != (tok_shards * t_l, kv_shards * w_l):
        raise ValueError(f"gathered {tuple(gathered.shape)} does not tile o {tuple(o_full.shape)}")
    o_full.view(tok_shards, t_l, kv_shards, w_l).copy_(gathered.view(kv_shards, tok_shards, t_l, w_l).permute(1, 2, 0, 3))
    return o_full


def all_gather_rows(out, local, group=None):
    """out [world, ...] <- every rank's `local`; one collective (NCCL: ncclAllGather; gloo for the CPU tests)."""
    import torch.distributed as dist
    if dist.get_backend(group) == "gloo":   # gloo has no flat all-gather into one tensor
        dist.all_gather(list(out.unbind(0)), local, group=group)
    else:
        dist.all_gather_into_tensor(out, local, group=group)


class HeadShardedPrefill:
    """The full layers' prefill chunk on `world` GPUs: this rank's kv heads and tokens through
    embla_attn_full_prefill, an all-gather of the per-head outputs on the same stream, the placement into
    token-major rows. The caller owns the pool (its kv heads only: `shard.n_kv_heads`) and the queries of its
    query heads and tokens."""

    def __init__(self, n_q_heads, n_kv_heads, act_dtype, n_tokens, max_context, world=1, rank=0, group=None, fused=False):
        from . import attn
        self.shard = prefill_partition(n_q_heads, n_kv_heads, n_tokens, world, rank)
        self.world, self.rank, self.group = world, rank, group
        self.ctx = attn.Attention(self.shard.n_q_heads, self.shard.n_kv_heads, act_dtype, 1, max_context)
        dt = self.ctx.torch_dtype
        self.fused = bool(fused) and world > 1
        self.width = n_q_heads * 128
        if self.fused:
            # every rank's output lives in symmetric memory: the peers' copies are mapped into this process, and the
            # kernel's epilogue stores this rank's rows into all of them
            import torch.distributed as dist
            import torch.distributed._symmetric_memory as symm
            self.o_full = symm.empty((n_tokens, self.width), dtype=dt, device=torch.device("cuda", torch.cuda.current_device()))
            self.o_full.zero_()
            self._symm = symm.rendezvous(self.o_full, group if group is not None else dist.group.WORLD)
            slab = (self.shard.token0 * self.width + self.shard.q_head0 * 128) * self.o_full.element_size()
            self.peer_ptrs = [int(self._symm.buffer_ptrs[r]) + slab for r in range(world) if r != rank]
            # this GPU's own place of the slab, as [1, T_l, ...] rows of the full width
            self.o_local = self.o_full[self.shard.token0:self.shard.token0 + self.shard.n_tokens,
                                       self.shard.q_head0 * 128:(self.shard.q_head0 + self.shard.n_q_heads) * 128].unsqueeze(0)
            self.gathered = None
            return
        self.o_full = torch.zeros(n_tokens, n_q_heads * 128, dtype=dt, device="cuda")
        if world == 1:                      # one GPU: the kernel writes the token-major output itself
            self.o_local, self.gathered = self.o_full.unsqueeze(0), None
            return
        self.o_local = torch.zeros(1, self.shard.n_tokens, self.shard.n_q_heads * 128, dtype=dt, device="cuda")
        self.gathered = torch.zeros(world, self.shard.n_tokens, self.shard.n_q_heads * 128, dtype=dt, device="cuda")

    def attend(self, pool, block_table, layer, pos0, q_local, gains=None):
        """The local kernel only: o_local [1][T_l][hq_l * 128]. pos0 = the position of THIS rank's first token."""
        from . import attn
        if self.fused:
            attn.full_prefill_scatter(self.ctx, pool, block_table, layer, pos0, q_local, self.o_local, self.peer_ptrs, self.width,
                                      gains=gains)
        else:
            attn.full_prefill(self.ctx, pool, block_table, layer, pos0, q_local, self.o_local, gains=gains)
        return self.o_local

    def combine(self):
        """All-gather of the per-head outputs and their placement: o_full [T][Hq * 128]. Fused: the rows are already in
        every GPU's output once every rank's kernel has finished, which one barrier across the GPUs establishes (a caller
        that reuses the output must also keep a peer from overwriting it while it is still read: another barrier, or two
        outputs in turn)."""
        if self.fused:
            self._symm.barrier()
            return self.o_full
        if self.world == 1:
            return self.o_full
        all_gather_rows(self.gathered, self.o_local[0], self.group)
        return place_heads(self.gathered, self.o_full, self.shard.kv_shards, self.shard.tok_shards)

    def run(self, pool, block_table, layer, pos0, q_local, gains=None):
        self.attend(pool, block_table, layer, pos0, q_local, gains)
        return self.combine()

    def close(self):
        self.ctx.close()


def max_over_ranks(value, device="cpu", group=None):
    """MAX of a python float over the ranks of the default (or given) process group."""
    import torch.distributed as dist
    t = torch.tensor([float(value)], device=device)
    if dist.is_available() and dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
