"""The head-sharded prefill chunk on two GPUs of one box, one process a GPU over NCCL: the kernel that stores its rows into
both GPUs' outputs (symmetric memory) against the all-gather path and against the CPU oracle. Skipped on a box with one GPU;
the partition and placement alone are covered on CPU (tests/test_sharding.py) and the scatter epilogue on one device
(tests/test_prefill_sharded_gpu.py)."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

T, P0, HQ, HKV, SEED = 512, 3000, 16, 4, 41


def _rank_main(rank, world, port, out_dir):
    import torch
    import torch.distributed as dist
    from embla_metal_b200 import attn, shard
    from oracle import oracle as orc
    from tests import util
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        rng = np.random.default_rng(SEED)               # every rank draws the same chunk and cache
        qb = orc.to_bits(rng.standard_normal((T, HQ, 128)), orc.BF16)
        k, ks, v, vs = util.int8_cache(rng, HKV, P0 + T, True)
        outs = {}
        for fused in (False, True):
            hsp = shard.HeadShardedPrefill(HQ, HKV, orc.BF16, T, P0 + T, world, rank, fused=fused)
            sh = hsp.shard
            S_l = P0 + sh.token0 + sh.n_tokens
            npg = (S_l + 127) // 128
            pool = attn.KVPool(1, sh.n_kv_heads, npg, attn.KV_INT8, attn.SCALE_F16)
            ids = np.arange(npg, dtype=np.int32)
            hs = slice(sh.kv_head0, sh.kv_head0 + sh.n_kv_heads)
            util.fill_pool(pool, 0, ids, k[hs, :S_l], ks[hs, :S_l], v[hs, :S_l], vs[hs, :S_l])
            q_l = qb[sh.token0:sh.token0 + sh.n_tokens, sh.q_head0:sh.q_head0 + sh.n_q_heads]
            qt = util.act_tensor(np.ascontiguousarray(q_l).reshape(1, sh.n_tokens, sh.n_q_heads * 128), orc.BF16)
            o = hsp.run(pool, torch.from_numpy(ids[None]).cuda(), 0,
                        torch.tensor([P0 + sh.token0], dtype=torch.int32, device="cuda"), qt)
            torch.cuda.synchronize()
            hsp.ctx.check()
            dist.barrier()
            outs[fused] = o.clone()
            pool.close()
            hsp.close()
        same = torch.equal(outs[True].view(torch.int16), outs[False].view(torch.int16))
        msg = "ok" if same else "fused and all-gather outputs differ"
        if same and rank == 0:
            r0, rstep = 3, 29
            _, want = orc.full_prefill(qb, orc.BF16, k, ks, v, vs, P0, r0=r0, rstep=rstep, nthreads=8, want_f32=True)
            got = orc.from_bits(util.act_bits(outs[True]), orc.BF16).reshape(T, HQ, 128)
            ok, why = util.close_stored(got[r0::rstep], want[r0::rstep], util.BF16_STEP)
            msg = "ok" if ok else why
        open(os.path.join(out_dir, f"rank{rank}.txt"), "w").write(msg)
    finally:
        dist.destroy_process_group()


def test_fused_prefill_on_two_gpus(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    port = 29600 + os.getpid() % 300
    mp.spawn(_rank_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for rank in range(2):
        assert open(tmp_path / f"rank{rank}.txt").read() == "ok"
