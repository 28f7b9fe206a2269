"""GPU parity of the full-layer decode kernel and the quantised append against the CPU oracle,
through the C ABI."""
import numpy as np
import pytest

from oracle import oracle as orc
from tests import util

pytestmark = pytest.mark.gpu


def _run_full(S_list, Hq, Hkv, dtype, scale_f16, gains=False, want_scores=False, seed=0, shuffle=True):
    import torch
    from embla_metal_b200 import attn
    rng = np.random.default_rng(seed)
    B = len(S_list)
    maxS = max(S_list)
    npg = (maxS + 127) // 128
    ctx = attn.Attention(Hq, Hkv, dtype, max_batch=B, max_context=npg * 128)
    pool = attn.KVPool(2, Hkv, B * npg + 3, attn.KV_INT8, attn.SCALE_F16 if scale_f16 else attn.SCALE_F32)
    layer = 1
    ids = rng.permutation(B * npg + 3) if shuffle else np.arange(B * npg + 3)
    table = ids[:B * npg].reshape(B, npg).astype(np.int32)
    q = rng.standard_normal((B, Hq, 128)).astype(np.float32)
    qb = orc.to_bits(q, dtype)
    g = None
    if gains:
        g = (orc.to_bits(rng.standard_normal(128) * 0.1, dtype), orc.to_bits(rng.standard_normal(128) * 0.1, dtype))
    want_o, want_sc, caches = [], [], []
    for b, S in enumerate(S_list):
        k, ks, v, vs = util.int8_cache(rng, Hkv, S, scale_f16)
        util.fill_pool(pool, layer, table[b], k, ks, v, vs)
        o, sc = orc.full_decode(qb[b], dtype, k, ks, v, vs, S, gains=g, want_scores=want_scores)
        want_o.append(orc.from_bits(o, dtype))
        want_sc.append(sc)
    qt = util.act_tensor(qb.reshape(B, Hq * 128), dtype)
    ot = torch.zeros_like(qt)
    gt = None if g is None else (util.act_tensor(g[0], dtype), util.act_tensor(g[1], dtype))
    sct = torch.full((B, Hkv, npg * 128), -7.0, device="cuda") if want_scores else None
    tbl = torch.from_numpy(table).cuda()
    lens = torch.tensor(S_list, dtype=torch.int32, device="cuda")
    ctx.full_decode(pool, tbl, lens, layer, qt, ot, gains=gt, scores=sct, max_seq_len=maxS)
    ctx.check()
    got = orc.from_bits(util.act_bits(ot), dtype).reshape(B, Hq, 128)
    # run twice: the split combine must be deterministic
    ot2 = torch.zeros_like(qt)
    ctx.full_decode(pool, tbl, lens, layer, qt, ot2, gains=gt, scores=sct, max_seq_len=maxS)
    torch.cuda.synchronize()
    assert torch.equal(ot.view(torch.int16), ot2.view(torch.int16))
    for b, S in enumerate(S_list):
        ok, msg = util.close(got[b], want_o[b])
        assert ok, f"seq {b} S={S}: {msg}"
        if want_scores:
            gs = sct[b, :, :S].cpu().numpy()
            assert np.array_equal(gs.view(np.uint32), want_sc[b][:, :S].view(np.uint32)), f"scores differ, seq {b} S={S}"
            assert float(sct[b, :, S:].min()) == -7.0 if S < npg * 128 else True
    pool.close()
    ctx.close()


def test_config0_full_decode():
    # benchmark configuration 0: 16 q / 4 kv heads, context 1024, fp16 q, int8 K/V, fp16 scales, seed 0
    _run_full([1024], 16, 4, orc.F16, True, seed=0)


@pytest.mark.parametrize("S", [1, 2, 127, 128, 129, 1151, 1152, 1153, 4096])
def test_edge_lengths(S):
    _run_full([S], 16, 4, orc.F16, True, seed=S)


def test_reference_shape_bf16_gains_fp32_scales():
    # the reference's own shape: 2 kv heads (8 query heads each), bf16, fp32 scales, fused head norm
    _run_full([1500], 16, 2, orc.BF16, False, gains=True, seed=5)


def test_ragged_batch():
    _run_full([700, 1, 3000, 129, 2048, 5], 16, 4, orc.F16, True, seed=7)


def test_scores_bit_exact():
    _run_full([1400, 130], 16, 4, orc.F16, True, want_scores=True, seed=11)
    _run_full([1300], 16, 2, orc.BF16, False, gains=True, want_scores=True, seed=12)


def test_context_32k():
    _run_full([32768], 16, 4, orc.F16, True, seed=3)


def test_kv_append_bit_exact():
    import torch
    from embla_metal_b200 import attn
    rng = np.random.default_rng(21)
    for dtype, scale_f16, Hkv in ((orc.BF16, False, 2), (orc.F16, True, 4)):
        B, T = 3, 37
        pos0 = np.array([0, 120, 250], np.int32)
        npg = 4
        ctx = attn.Attention(16, Hkv, dtype, max_batch=B, max_context=npg * 128)
        pool = attn.KVPool(1, Hkv, B * npg, attn.KV_INT8, attn.SCALE_F16 if scale_f16 else attn.SCALE_F32)
        table = rng.permutation(B * npg).reshape(B, npg).astype(np.int32)
        k = rng.standard_normal((B, T, Hkv, 128)).astype(np.float32) * 3
        v = rng.standard_normal((B, T, Hkv, 128)).astype(np.float32)
        k[1, 3, 0] = 0.0
        v[2, 5, 1] = 0.0
        kb, vb = orc.to_bits(k, dtype), orc.to_bits(v, dtype)
        ctx.kv_append(pool, torch.from_numpy(table).cuda(), 0, torch.from_numpy(pos0).cuda(),
                      util.act_tensor(kb.reshape(B, T, Hkv * 128), dtype), util.act_tensor(vb.reshape(B, T, Hkv * 128), dtype))
        torch.cuda.synchronize()
        raw = pool.raw().cpu().numpy()
        ssz = 2 if scale_f16 else 4
        sdt = np.float16 if scale_f16 else np.float32
        for b in range(B):
            for t in range(T):
                pos = pos0[b] + t
                blk, row = table[b, pos // 128], pos % 128
                for h in range(Hkv):
                    page = raw[blk, 0, h]
                    kc, ksc = orc.quantize_rows(kb[b, t, h], dtype, norm=True, scale_f16=scale_f16)
                    vc, vsc = orc.quantize_rows(vb[b, t, h], dtype, norm=False, scale_f16=scale_f16)
                    assert np.array_equal(page[row * 128:(row + 1) * 128].view(np.int8), kc[0])
                    assert np.array_equal(page[16384 + row * 128:16384 + (row + 1) * 128].view(np.int8), vc[0])
                    gks = page[32768 + row * ssz:32768 + (row + 1) * ssz].view(sdt)[0]
                    gvs = page[32768 + 128 * ssz + row * ssz:32768 + 128 * ssz + (row + 1) * ssz].view(sdt)[0]
                    assert np.float32(gks) == ksc[0] and np.float32(gvs) == vsc[0]
        pool.close()
        ctx.close()


@pytest.mark.parametrize("dtype,scale_f16,Hkv,norm_k", [(orc.F16, True, 4, False), (orc.BF16, False, 2, True)])
def test_fused_append_equals_append_then_decode(dtype, scale_f16, Hkv, norm_k):
    """embla_attn_full_step writes the same page bytes and outputs as embla_kv_append + embla_attn_full_decode, with and
    without scores, for positions at the start, inside and at the end of a page and for split and unsplit key ranges."""
    import torch
    from embla_metal_b200 import attn
    rng = np.random.default_rng(31)
    S_list = [1, 2, 128, 129, 300, 1024, 4097, 9000]
    B, Hq = len(S_list), 16
    npg = (max(S_list) + 127) // 128
    ctx = attn.Attention(Hq, Hkv, dtype, max_batch=B, max_context=npg * 128)
    pools = [attn.KVPool(1, Hkv, B * npg, attn.KV_INT8, attn.SCALE_F16 if scale_f16 else attn.SCALE_F32) for _ in range(2)]
    table = torch.from_numpy(rng.permutation(B * npg).reshape(B, npg).astype(np.int32)).cuda()
    fill = torch.from_numpy(rng.integers(0, 256, pools[0].raw().shape, dtype=np.uint8)).cuda()
    for pool in pools:
        raw = pool.raw()
        raw.copy_(fill)
        sc = raw[..., 32768:].view(torch.float16 if scale_f16 else torch.float32)
        sc.copy_(torch.rand(sc.shape, device="cuda") * 0.015 + 0.005)
    pools[1].raw().copy_(pools[0].raw())
    lens = torch.tensor(S_list, dtype=torch.int32, device="cuda")
    q = util.act_tensor(orc.to_bits(rng.standard_normal((B, Hq * 128)), dtype), dtype)
    k = util.act_tensor(orc.to_bits(rng.standard_normal((B, Hkv * 128)) * 2, dtype), dtype)
    v = util.act_tensor(orc.to_bits(rng.standard_normal((B, Hkv * 128)), dtype), dtype)
    for want_scores in (False, True):
        o0, o1 = torch.zeros_like(q), torch.zeros_like(q)
        sc0 = torch.zeros(B, Hkv, npg * 128, device="cuda") if want_scores else None
        sc1 = torch.zeros_like(sc0) if want_scores else None
        ctx.kv_append(pools[0], table, 0, lens - 1, k.view(B, 1, -1), v.view(B, 1, -1), norm_k=norm_k)
        ctx.full_decode(pools[0], table, lens, 0, q, o0, scores=sc0, max_seq_len=max(S_list))
        ctx.full_step(pools[1], table, lens, 0, q, k, v, o1, scores=sc1, max_seq_len=max(S_list), norm_k=norm_k)
        ctx.check()
        assert torch.equal(pools[0].raw(), pools[1].raw()), "the fused append wrote other bytes"
        assert torch.equal(o0.view(torch.int16), o1.view(torch.int16)), "outputs differ"
        if want_scores:
            for b, S in enumerate(S_list):
                assert torch.equal(sc0[b, :, :S], sc1[b, :, :S]), f"scores of sequence {b} differ"
    for pool in pools:
        pool.close()
    ctx.close()
