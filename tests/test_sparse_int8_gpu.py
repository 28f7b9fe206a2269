"""The reference's own block structure on the GPU: a full layer attends over its int8 cache and emits key scores,
the selection takes the top 1024 + 128 latest rows, and the following sparse layer attends those rows of the SAME
int8 cache with its own query (Sources/EmblaMetal/Engine.swift:461-462, 796-827). Checked against the CPU oracle."""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as orc
from tests import util

pytestmark = pytest.mark.gpu


def _sparse_int8(attn, ctx, pool, tbl, lens, layer, q, o, idx, gains, max_seq_len):
    import torch
    view = attn.Attention.view(tbl, lens, layer, max_seq_len)
    qd = attn.Attention.query(q, gains)
    attn._check(attn.lib().embla_attn_sparse_decode_int8(ctx.handle, pool.handle, C.byref(view), C.byref(qd),
                                                         None if idx is None else C.c_void_p(idx.data_ptr()),
                                                         C.c_void_p(o.data_ptr()), C.c_int64(o.stride(0)),
                                                         C.c_void_p(torch.cuda.current_stream().cuda_stream)))


def _block(S, Hq, Hkv, dtype, scale_f16, seed, gains):
    import torch
    from embla_metal_b200 import attn
    rng = np.random.default_rng(seed)
    npg = (S + 127) // 128
    ctx = attn.Attention(Hq, Hkv, dtype, 1, npg * 128)
    pool = attn.KVPool(1, Hkv, npg + 2, attn.KV_INT8, attn.SCALE_F16 if scale_f16 else attn.SCALE_F32)
    ids = rng.permutation(npg + 2)[:npg].astype(np.int32)
    k, ks, v, vs = util.int8_cache(rng, Hkv, S, scale_f16)
    util.fill_pool(pool, 0, ids, k, ks, v, vs)
    q_full = orc.to_bits(rng.standard_normal((Hq, 128)), dtype)
    q_sparse = orc.to_bits(rng.standard_normal((Hq, 128)) * 2.0, dtype)
    g = None
    if gains:
        g = (orc.to_bits(rng.standard_normal(128) * 0.1, dtype), orc.to_bits(rng.standard_normal(128) * 0.1, dtype))
    gt = None if g is None else tuple(util.act_tensor(x, dtype) for x in g)
    tbl = torch.from_numpy(ids[None]).cuda()
    lens = torch.tensor([S], dtype=torch.int32, device="cuda")
    qf = util.act_tensor(q_full.reshape(1, -1), dtype)
    of = torch.zeros_like(qf)
    sc = torch.zeros(1, Hkv, npg * 128, device="cuda")
    ctx.full_decode(pool, tbl, lens, 0, qf, of, gains=gt, scores=sc, max_seq_len=S)
    want_of, want_sc = orc.full_decode(q_full, dtype, k, ks, v, vs, S, gains=g, want_scores=True)
    idx_t, want_idx = None, None
    if S > 1152:
        idx_t = torch.zeros(1, Hkv, 1152, dtype=torch.int32, device="cuda")
        ctx.select_keys(sc, lens, idx_t, max_seq_len=S)
        want_idx = orc.select_keys(want_sc, S)
        assert np.array_equal(idx_t[0].cpu().numpy().view(np.uint32), want_idx), "selected rows differ"
    qs = util.act_tensor(q_sparse.reshape(1, -1), dtype)
    os_ = torch.zeros_like(qs)
    _sparse_int8(attn, ctx, pool, tbl, lens, 0, qs, os_, idx_t, gt, S)
    ctx.check()
    want_os = orc.from_bits(orc.sparse_decode(q_sparse, dtype, k, ks, v, vs, S, idx=want_idx, kv_kind=0, gains=g), dtype)
    got_os = orc.from_bits(util.act_bits(os_), dtype).reshape(Hq, 128)
    step = util.BF16_STEP if dtype == orc.BF16 else 0.0
    ok, msg = util.close(got_os, want_os, out_ulp=step, rel_rms=4e-3 if dtype == orc.BF16 else util.REL_RMS)
    assert ok, f"sparse over int8, S={S}: {msg}"
    pool.close()
    ctx.close()


@pytest.mark.parametrize("S", [1, 100, 512, 513, 1152, 1153, 5000])
def test_block_fp16(S):
    _block(S, 16, 4, orc.F16, True, seed=40 + S, gains=False)


def test_block_reference_shape():
    # 2 kv heads x 8 query heads, bf16, fp32 scales, head norm with both gains — the reference's own shape
    _block(3000, 16, 2, orc.BF16, False, seed=7, gains=True)
    _block(900, 16, 2, orc.BF16, False, seed=8, gains=True)
