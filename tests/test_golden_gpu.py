"""The CUDA kernels against the committed golden fixtures (tests/golden/attention_golden.npz), through
the C ABI: bytes, scores and index lists bit for bit, attention outputs within tolerance."""
import os

import numpy as np
import pytest

from oracle import oracle as orc
from tests import util

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "attention_golden.npz")


@pytest.fixture(scope="module")
def g():
    return np.load(GOLD)


def _full(g, pre, dtype, scale_f16, gains):
    import torch
    from embla_metal_b200 import attn
    q, k, v, ks, vs = (g[pre + n] for n in ("_q", "_k", "_v", "_ks", "_vs"))
    Hq, Hkv, S = q.shape[0], k.shape[0], k.shape[1]
    npg = (S + 127) // 128
    ctx = attn.Attention(Hq, Hkv, dtype, 1, npg * 128)
    pool = attn.KVPool(1, Hkv, npg, attn.KV_INT8, attn.SCALE_F16 if scale_f16 else attn.SCALE_F32)
    util.fill_pool(pool, 0, list(range(npg)), k, ks, v, vs)
    tbl = torch.arange(npg, dtype=torch.int32, device="cuda")[None].contiguous()
    lens = torch.tensor([S], dtype=torch.int32, device="cuda")
    qt = util.act_tensor(q.reshape(1, -1), dtype)
    ot = torch.zeros_like(qt)
    sc = torch.zeros(1, Hkv, npg * 128, device="cuda")
    gt = None if gains is None else tuple(util.act_tensor(x, dtype) for x in gains)
    ctx.full_decode(pool, tbl, lens, 0, qt, ot, gains=gt, scores=sc, max_seq_len=S)
    ctx.check()
    ok, msg = util.close(orc.from_bits(util.act_bits(ot), dtype).reshape(Hq, 128), orc.from_bits(g[pre + "_o"], dtype))
    assert ok, msg
    assert np.array_equal(sc[0, :, :S].cpu().numpy().view(np.uint32), g[pre + "_scores"][:, :S].view(np.uint32))
    pool.close()
    ctx.close()


def test_full_decode_golden(g):
    _full(g, "full", orc.F16, True, None)
    _full(g, "ref", orc.BF16, False, (g["ref_g1"], g["ref_g2"]))


def test_quantised_append_golden(g):
    import torch
    from embla_metal_b200 import attn
    x = g["quant_x"]                                  # 12 rows: 3 tokens x 4 kv heads
    ctx = attn.Attention(16, 4, orc.BF16, 1, 128)
    pool = attn.KVPool(1, 4, 1, attn.KV_INT8, attn.SCALE_F32)
    rows = util.act_tensor(x.reshape(1, 3, 4 * 128), orc.BF16)
    tbl = torch.zeros((1, 1), dtype=torch.int32, device="cuda")
    ctx.kv_append(pool, tbl, 0, torch.tensor([5], dtype=torch.int32, device="cuda"), rows, rows, norm_k=True)
    torch.cuda.synchronize()
    raw = pool.raw().cpu().numpy()[0, 0]              # [4 heads, page]
    for t in range(3):
        for h in range(4):
            r = 5 + t
            i = t * 4 + h
            assert np.array_equal(raw[h, r * 128:(r + 1) * 128].view(np.int8), g["quant_codes_norm"][i])
            assert np.array_equal(raw[h, 16384 + r * 128:16384 + (r + 1) * 128].view(np.int8), g["quant_codes_plain"][i])
            assert raw[h, 32768 + 4 * r:32768 + 4 * r + 4].view(np.float32)[0] == g["quant_scales_norm"][i]
            assert raw[h, 32768 + 512 + 4 * r:32768 + 512 + 4 * r + 4].view(np.float32)[0] == g["quant_scales_plain"][i]
    pool.close()
    ctx.close()


def test_selection_golden(g):
    import torch
    from embla_metal_b200 import attn
    sc = g["sel_scores"]
    Hkv, S = sc.shape
    ctx = attn.Attention(2 * Hkv, Hkv, orc.F16, 1, S)
    idx = torch.zeros(1, Hkv, 1152, dtype=torch.int32, device="cuda")
    ctx.select_keys(torch.from_numpy(sc[None]).cuda(), torch.tensor([S], dtype=torch.int32, device="cuda"), idx, max_seq_len=S)
    torch.cuda.synchronize()
    assert np.array_equal(idx[0].cpu().numpy().view(np.uint32), g["sel_idx"])
    ctx.close()


@pytest.mark.parametrize("name", ["sparse_short", "sparse_sel"])
def test_sparse_golden(g, name):
    import torch
    from embla_metal_b200 import attn
    q, kb, vb = g[name + "_q"], g[name + "_k"], g[name + "_v"]
    Hq, Hkv, S = q.shape[0], kb.shape[0], kb.shape[1]
    npg = (S + 127) // 128
    ctx = attn.Attention(Hq, Hkv, orc.F16, 1, npg * 128)
    pool = attn.KVPool(1, Hkv, npg, attn.KV_16BIT)
    tbl = torch.arange(npg, dtype=torch.int32, device="cuda")[None].contiguous()
    pos0 = torch.zeros(1, dtype=torch.int32, device="cuda")
    # the rows go in through the 16-bit append (a copy), as a caller would write them
    ctx.kv_append(pool, tbl, 0, pos0, util.act_tensor(kb.transpose(1, 0, 2).reshape(1, S, Hkv * 128), orc.F16),
                  util.act_tensor(vb.transpose(1, 0, 2).reshape(1, S, Hkv * 128), orc.F16), norm_k=False)
    lens = torch.tensor([S], dtype=torch.int32, device="cuda")
    qt = util.act_tensor(q.reshape(1, -1), orc.F16)
    sc = torch.zeros(1, Hkv, npg * 128, device="cuda")
    ctx.score_keys(pool, tbl, lens, 0, qt, sc, max_seq_len=S)
    assert np.array_equal(sc[0, :, :S].cpu().numpy().view(np.uint32), g[name + "_scores"][:, :S].view(np.uint32))
    idx = None
    if S > 1152:
        idx = torch.zeros(1, Hkv, 1152, dtype=torch.int32, device="cuda")
        ctx.select_keys(sc, lens, idx, max_seq_len=S)
        assert np.array_equal(idx[0].cpu().numpy().view(np.uint32), g[name + "_idx"])
    ot = torch.zeros_like(qt)
    ctx.sparse_decode(pool, tbl, lens, 0, qt, ot, idx=idx, max_seq_len=S)
    ctx.check()
    ok, msg = util.close(orc.from_bits(util.act_bits(ot), orc.F16).reshape(Hq, 128), orc.from_bits(g[name + "_o"], orc.F16))
    assert ok, msg
    pool.close()
    ctx.close()


def test_sliding_golden(g):
    import torch
    from embla_metal_b200 import attn
    hk, hv = g["slide_hist_k"], g["slide_hist_v"]          # [T, Hkv, 128]
    T, Hkv = hk.shape[0], hk.shape[1]
    q = g["slide_q"]
    Hq = q.shape[1]
    RING = g["slide_ring_k"].shape[1]
    ctx = attn.Attention(Hq, Hkv, orc.BF16, 1, 1024)
    ring = attn.Ring(1, Hkv, RING, 128, torch.bfloat16)
    kg, qg = util.act_tensor(g["slide_kg"], orc.BF16), util.act_tensor(g["slide_qg"], orc.BF16)
    # the ring holds RING slots: write the history in chunks no longer than the ring, like prefill chunks
    for t0 in range(0, T, 128):
        n = min(128, T - t0)
        ctx.sliding_write(ring, torch.tensor([t0], dtype=torch.int32, device="cuda"),
                          util.act_tensor(hk[t0:t0 + n].reshape(1, n, Hkv * 128), orc.BF16),
                          util.act_tensor(hv[t0:t0 + n].reshape(1, n, Hkv * 128), orc.BF16), kgain=kg)
    torch.cuda.synchronize()
    got_k = orc.from_bits(util.act_bits(ring.k[0]), orc.BF16)
    want_k = orc.from_bits(g["slide_ring_k"], orc.BF16)
    # norm + RoPE in the oracle's operation order; sin/cos may differ by an ulp, so allow one bf16 step
    assert np.abs(got_k - want_k).max() <= 2.0 ** -7 * np.abs(want_k).max()
    assert (util.act_bits(ring.k[0]) == g["slide_ring_k"]).mean() > 0.999
    assert np.array_equal(util.act_bits(ring.v[0]), g["slide_ring_v"])
    qt = util.act_tensor(q.reshape(1, -1), orc.BF16)
    ot = torch.zeros_like(qt)
    ctx.sliding_decode(ring, torch.tensor([T], dtype=torch.int32, device="cuda"), qt, ot, qgain=qg)
    ctx.check()
    ok, msg = util.close(orc.from_bits(util.act_bits(ot), orc.BF16).reshape(Hq, 128), orc.from_bits(g["slide_o"][0], orc.BF16),
                         max_abs=4e-3, rel_rms=4e-3)   # one bf16 output step is 2^-9 relative
    assert ok, msg
    ctx.close()
