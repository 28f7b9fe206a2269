"""Parity where the scores are large. The other tests draw q ~ N(0, 1) with gains near 0, so |q·k| / sqrt(D) stays
below about 6. In the reference's own arrangement q is head-normed with gains (1 + g1)(1 + g2) and k is normed, so a
key aligned with a query scores sqrt(128) (1 + g)^2: 45 at gains of 1, 180 at gains of 3, and the ReLU² weight is its
square. The reference keeps those weights in fp32 (attn_nax.metal:11, attention.metal:143-145); the CUDA kernels keep
some of them in fp16, which these cases pin: reference-native shape (2 kv heads x 8 query heads, bf16, fp32 scales,
fused head norm), keys quantised from normed rows over the quantiser's full range, a few of them aligned with queries.
"""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as orc
from tests import util

pytestmark = pytest.mark.gpu
HQ, HKV, DT = 16, 2, orc.BF16


def _gains(rng, g):
    return (orc.to_bits(g + rng.standard_normal(128) * 0.02, DT), orc.to_bits(g + rng.standard_normal(128) * 0.02, DT))


def _normed(x, gains):
    """fp32 approximation of head_norm with both gains (only used to aim keys at queries)."""
    x = np.asarray(x, np.float32)
    r = 1.0 / np.sqrt((x * x).mean(-1, keepdims=True) + 1.1920929e-7)
    out = x * r
    for gb in gains:
        out = out * (1.0 + orc.from_bits(gb, DT))
    return out


def _cache_aligned(rng, S, q_rows, where):
    """int8 cache [HKV, S, 128] quantised from normed rows (as kv_append does); key where[i] of the kv head of
    q_rows[i] = (head, vector) points along that query."""
    k_raw = rng.standard_normal((HKV, S, 128)).astype(np.float32)
    for (head, vec), pos in zip(q_rows, where):
        k_raw[head // (HQ // HKV), pos] = vec
    v_raw = rng.standard_normal((HKV, S, 128)).astype(np.float32)
    kc, ks = orc.quantize_rows(orc.to_bits(k_raw.reshape(-1, 128), DT), DT, norm=True)
    vc, vs = orc.quantize_rows(orc.to_bits(v_raw.reshape(-1, 128), DT), DT, norm=False)
    return kc.reshape(HKV, S, 128), ks.reshape(HKV, S), vc.reshape(HKV, S, 128), vs.reshape(HKV, S)


@pytest.mark.parametrize("gain", [1.0, 3.0])
def test_full_decode_and_shared_sparse_large_scores(gain):
    import torch
    from embla_metal_b200 import attn
    rng = np.random.default_rng(int(gain * 10))
    S = 3000
    npg = (S + 127) // 128
    g = _gains(rng, gain)
    q = rng.standard_normal((HQ, 128)).astype(np.float32)
    qb = orc.to_bits(q, DT)
    qn = _normed(orc.from_bits(qb, DT), g)
    aims = [(h, qn[h]) for h in (0, 3, 9, 15)]
    k, ks, v, vs = _cache_aligned(rng, S, aims, [5, 1500, 2990, 2999])
    ctx = attn.Attention(HQ, HKV, DT, 1, npg * 128)
    pool = attn.KVPool(1, HKV, npg, attn.KV_INT8, attn.SCALE_F32)
    ids = rng.permutation(npg).astype(np.int32)
    util.fill_pool(pool, 0, ids, k, ks, v, vs)
    tbl = torch.from_numpy(ids[None]).cuda()
    lens = torch.tensor([S], dtype=torch.int32, device="cuda")
    gt = tuple(util.act_tensor(x, DT) for x in g)
    qt = util.act_tensor(qb.reshape(1, -1), DT)
    ot = torch.zeros_like(qt)
    sc = torch.zeros(1, HKV, npg * 128, device="cuda")
    ctx.full_decode(pool, tbl, lens, 0, qt, ot, gains=gt, scores=sc, max_seq_len=S)
    ctx.check()
    want_o, want_sc = orc.full_decode(qb, DT, k, ks, v, vs, S, gains=g, want_scores=True)
    assert np.abs(want_sc).max() / np.sqrt(128.0) > 0.8 * np.sqrt(128.0) * (1 + gain) ** 2, "the case lost its large scores"
    assert np.array_equal(sc[0, :, :S].cpu().numpy().view(np.uint32), want_sc[:, :S].view(np.uint32))
    got = orc.from_bits(util.act_bits(ot), DT).reshape(HQ, 128)
    assert np.isfinite(got).all()
    ok, msg = util.close(got, orc.from_bits(want_o, DT), out_ulp=util.BF16_STEP)
    assert ok, f"full decode, gains {gain}: {msg}"
    # the sparse layer that shares this cache: softmax over the selected rows, scores of the same size
    idx = torch.zeros(1, HKV, 1152, dtype=torch.int32, device="cuda")
    ctx.select_keys(sc, lens, idx, max_seq_len=S)
    want_idx = orc.select_keys(want_sc, S)
    assert np.array_equal(idx[0].cpu().numpy().view(np.uint32), want_idx)
    os_ = torch.zeros_like(qt)
    view = attn.Attention.view(tbl, lens, 0, S)
    qd = attn.Attention.query(qt, gt)
    attn._check(attn.lib().embla_attn_sparse_decode_int8(ctx.handle, pool.handle, C.byref(view), C.byref(qd),
                                                         C.c_void_p(idx.data_ptr()), C.c_void_p(os_.data_ptr()),
                                                         C.c_int64(os_.stride(0)), None))
    ctx.check()
    want_s = orc.from_bits(orc.sparse_decode(qb, DT, k, ks, v, vs, S, idx=want_idx, kv_kind=0, gains=g), DT)
    got_s = orc.from_bits(util.act_bits(os_), DT).reshape(HQ, 128)
    assert np.isfinite(got_s).all()
    ok, msg = util.close(got_s, want_s, out_ulp=util.BF16_STEP, rel_rms=4e-3)
    assert ok, f"sparse over the shared cache, gains {gain}: {msg}"
    pool.close()
    ctx.close()


@pytest.mark.parametrize("gain", [1.0, 3.0])
def test_full_prefill_large_scores(gain):
    import torch
    from embla_metal_b200 import attn
    rng = np.random.default_rng(100 + int(gain * 10))
    T, p0 = 300, 700
    S = p0 + T
    npg = (S + 127) // 128
    g = _gains(rng, gain)
    qb = orc.to_bits(rng.standard_normal((T, HQ, 128)), DT)
    qn = _normed(orc.from_bits(qb, DT), g)
    # query rows 0, 100, 299 (heads 1, 8, 14) each find an aligned key: far back, inside the chunk, and on the diagonal
    aims = [(1, qn[0, 1]), (8, qn[100, 8]), (14, qn[299, 14]), (14, qn[250, 14])]
    k, ks, v, vs = _cache_aligned(rng, S, aims, [3, p0 + 50, p0 + 299, 640])
    ctx = attn.Attention(HQ, HKV, DT, 1, npg * 128)
    pool = attn.KVPool(1, HKV, npg, attn.KV_INT8, attn.SCALE_F32)
    ids = rng.permutation(npg).astype(np.int32)
    util.fill_pool(pool, 0, ids, k, ks, v, vs)
    tbl = torch.from_numpy(ids[None]).cuda()
    gt = tuple(util.act_tensor(x, DT) for x in g)
    qt = util.act_tensor(qb.reshape(1, T, HQ * 128), DT)
    ot = torch.zeros_like(qt)
    attn.full_prefill(ctx, pool, tbl, 0, torch.tensor([p0], dtype=torch.int32, device="cuda"), qt, ot, gains=gt)
    ctx.check()
    got = orc.from_bits(util.act_bits(ot), DT).reshape(T, HQ, 128)
    assert np.isfinite(got).all(), "a weight or a row sum left fp16's range"
    _, want = orc.full_prefill(qb, DT, k, ks, v, vs, p0, gains=g, nthreads=8, want_f32=True)
    ok, msg = util.close_stored(got, want, util.BF16_STEP)
    assert ok, f"full prefill, gains {gain}: {msg}"
    pool.close()
    ctx.close()


@pytest.mark.parametrize("gain", [1.0, 3.0])
def test_sliding_decode_large_scores(gain):
    """Softmax layers: q and k both normed with a gain, so the scores' spread grows with (1 + g)^2 and the softmax is
    close to one-hot; exp(s - max) never leaves [0, 1]."""
    import torch
    from embla_metal_b200 import attn
    rng = np.random.default_rng(200 + int(gain * 10))
    Hq, Hkv, W, RING, pos = 16, 4, 128, 4096, 5000
    ctx = attn.Attention(Hq, Hkv, DT, max_batch=1, max_context=RING)
    ring = attn.Ring(1, Hkv, RING, W, torch.bfloat16)
    qg = orc.to_bits(gain + rng.standard_normal(128) * 0.02, DT)
    kg = orc.to_bits(gain + rng.standard_normal(128) * 0.02, DT)
    rk = np.zeros((Hkv, RING, 128), np.uint16)
    rv = np.zeros((Hkv, RING, 128), np.uint16)
    n_hist = RING - 1
    hk = orc.to_bits(rng.standard_normal((n_hist, Hkv, 128)), DT)
    hv = orc.to_bits(rng.standard_normal((n_hist, Hkv, 128)), DT)
    orc.sliding_write(hk, hv, DT, rk, rv, pos - n_hist, kgain=kg)
    ring.k.copy_(util.act_tensor(rk[None], DT))
    ring.v.copy_(util.act_tensor(rv[None], DT))
    q = orc.to_bits(rng.standard_normal((1, Hq, 128)), DT)
    knew = orc.to_bits(rng.standard_normal((1, Hkv, 128)), DT)
    vnew = orc.to_bits(rng.standard_normal((1, Hkv, 128)), DT)
    orc.sliding_write(knew, vnew, DT, rk, rv, pos, kgain=kg)
    want = orc.from_bits(orc.sliding_attend(q, DT, rk, rv, pos, W, qgain=qg), DT)[0]
    qkv = np.concatenate([q.reshape(1, -1), knew.reshape(1, -1), vnew.reshape(1, -1)], axis=1)
    row = util.act_tensor(qkv, DT)
    ot = torch.zeros(1, Hq * 128, dtype=torch.bfloat16, device="cuda")
    lens = torch.tensor([pos + 1], dtype=torch.int32, device="cuda")
    qd = attn.Query(row.data_ptr(), row.stride(0), 0, 1, util.act_tensor(qg, DT).data_ptr(), None)
    qg_t, kg_t = util.act_tensor(qg, DT), util.act_tensor(kg, DT)
    qd = attn.Query(row.data_ptr(), row.stride(0), 0, 1, qg_t.data_ptr(), None)
    attn._check(attn.lib().embla_attn_sliding_step(
        ctx.handle, C.byref(ring.desc), C.c_void_p(lens.data_ptr()), 1, C.byref(qd),
        C.c_void_p(row.data_ptr() + Hq * 128 * 2), C.c_void_p(row.data_ptr() + (Hq + Hkv) * 128 * 2), C.c_int64(row.stride(0)),
        0, C.c_void_p(kg_t.data_ptr()), C.c_void_p(ot.data_ptr()), C.c_int64(ot.stride(0)), None))
    ctx.check()
    got = orc.from_bits(util.act_bits(ot), DT).reshape(Hq, 128)
    assert np.isfinite(got).all()
    ok, msg = util.close(got, want, out_ulp=util.BF16_STEP, rel_rms=4e-3)
    assert ok, f"sliding step, gains {gain}: {msg}"
    ctx.close()
