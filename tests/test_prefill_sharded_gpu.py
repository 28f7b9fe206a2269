"""The head-sharded prefill path on one device: the shards that 2, 4 and 8 GPUs would compute are run one after
another, assembled as the all-gather leaves them (rank-major), placed token-major, and compared with the CPU oracle
on BASELINE config 3 (2048-token chunk after 30720 cached positions). The collective itself is covered by the 2-rank
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
