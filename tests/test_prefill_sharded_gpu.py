"""The head-sharded prefill path on one device: the shards that 2, 4 and 8 GPUs would compute are run one after
another, assembled as the all-gather leaves them (rank-major), placed token-major, and compared with the CPU oracle
on benchmark configuration 3 (2048-token chunk after 30720 cached positions). The collective itself is covered by the 2-rank
gloo test of the same placement (tests/test_sharding.py)."""
import numpy as np
import pytest

from oracle import oracle as orc
from tests import util

pytestmark = pytest.mark.gpu


def test_shards_assemble_to_the_single_gpu_result():
    import torch
    from embla_metal_b200 import attn, shard
    rng = np.random.default_rng(3)
    T, p0, Hq, Hkv, dtype = 2048, 30720, 16, 4, orc.BF16
    qb = orc.to_bits(rng.standard_normal((T, Hq, 128)), dtype)
    k, ks, v, vs = util.int8_cache(rng, Hkv, p0 + T, True)
    r0, rstep = 5, 37
    _, want = orc.full_prefill(qb, dtype, k, ks, v, vs, p0, r0=r0, rstep=rstep, nthreads=8, want_f32=True)
    for world in (2, 4, 8):
        gathered = None
        for rank in range(world):
            sh = shard.prefill_partition(Hq, Hkv, T, world, rank)
            hsp = shard.HeadShardedPrefill(Hq, Hkv, dtype, T, p0 + T, world, rank)
            S_l = p0 + sh.token0 + sh.n_tokens                      # keys this rank's tokens can see
            npg = (S_l + 127) // 128
            pool = attn.KVPool(1, sh.n_kv_heads, npg, attn.KV_INT8, attn.SCALE_F16)
            ids = np.arange(npg, dtype=np.int32)
            hs = slice(sh.kv_head0, sh.kv_head0 + sh.n_kv_heads)
            util.fill_pool(pool, 0, ids, k[hs, :S_l], ks[hs, :S_l], v[hs, :S_l], vs[hs, :S_l])
            q_l = qb[sh.token0:sh.token0 + sh.n_tokens, sh.q_head0:sh.q_head0 + sh.n_q_heads]
            qt = util.act_tensor(np.ascontiguousarray(q_l).reshape(1, sh.n_tokens, sh.n_q_heads * 128), dtype)
            o_l = hsp.attend(pool, torch.from_numpy(ids[None]).cuda(), 0,
                             torch.tensor([p0 + sh.token0], dtype=torch.int32, device="cuda"), qt)
            hsp.ctx.check()
            if gathered is None:
                gathered = torch.zeros(world, sh.n_tokens, sh.n_q_heads * 128, dtype=o_l.dtype, device="cuda")
            gathered[rank].copy_(o_l[0])
            torch.cuda.synchronize()
            pool.close()
            hsp.close()
        sh = shard.prefill_partition(Hq, Hkv, T, world, 0)
        o = shard.place_heads(gathered, torch.zeros(T, Hq * 128, dtype=gathered.dtype, device="cuda"), sh.kv_shards, sh.tok_shards)
        got = orc.from_bits(util.act_bits(o), dtype).reshape(T, Hq, 128)
        ok, msg = util.close_stored(got[r0::rstep], want[r0::rstep], util.BF16_STEP)
        assert ok, f"{world} shards: {msg}"


def test_scatter_epilogue_writes_every_copy():
    """embla_attn_full_prefill_scatter with its "peers" on the same device: the kernel's epilogue puts the shard's rows at
    their place in three token-major outputs, both through the direct epilogue (many units) and through the split-KV
    combine (few units), and they equal the plain call's rows bit for bit."""
    import torch
    from embla_metal_b200 import attn
    for T, p0, seed in ((300, 1000, 31), (200, 12000, 32)):          # second case: pages of a unit split over CTAs
        rng = np.random.default_rng(seed)
        Hq_all, Hq, Hkv, dtype = 16, 8, 2, orc.BF16                    # this "rank": query heads 4..11 of 16
        q = orc.to_bits(rng.standard_normal((T, Hq, 128)), dtype)
        k, ks, v, vs = util.int8_cache(rng, Hkv, p0 + T, True)
        npg = (p0 + T + 127) // 128
        ctx = attn.Attention(Hq, Hkv, dtype, 1, npg * 128)
        pool = attn.KVPool(1, Hkv, npg, attn.KV_INT8, attn.SCALE_F16)
        ids = np.arange(npg, dtype=np.int32)
        util.fill_pool(pool, 0, ids, k, ks, v, vs)
        tbl = torch.from_numpy(ids[None]).cuda()
        qt = util.act_tensor(q.reshape(1, T, Hq * 128), dtype)
        pos0 = torch.tensor([p0], dtype=torch.int32, device="cuda")
        plain = torch.zeros_like(qt)
        attn.full_prefill(ctx, pool, tbl, 0, pos0, qt, plain)
        width, head0, tok0, T_all = Hq_all * 128, 4, 64, T + 100
        outs = [torch.full((T_all, width), 7.0, dtype=torch.bfloat16, device="cuda") for _ in range(3)]
        place = lambda o: o[tok0:tok0 + T, head0 * 128:(head0 + Hq) * 128]
        peers = [o.data_ptr() + (tok0 * width + head0 * 128) * 2 for o in outs[1:]]
        attn.full_prefill_scatter(ctx, pool, tbl, 0, pos0, qt, place(outs[0]).unsqueeze(0), peers, width)
        ctx.check()
        for o in outs:
            assert torch.equal(place(o).view(torch.int16), plain[0].view(torch.int16))
            rest = o.clone()
            place(rest).fill_(7.0)
            assert bool((rest == 7.0).all()), "rows outside the slab were touched"
        pool.close()
        ctx.close()
