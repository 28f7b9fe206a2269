"""GPU parity of the q/k/v producer: the reference's 4-bit stacked GEMV (gemv / GemvRows, Sources/EmblaMetal/Kernels/
gemv.metal:37-92, common.metal:105-152) against its CPU restatement (the products are exact on both sides, the fp32 sums
differ in order only: outputs equal or one step of the storage dtype apart), and its fused epilogue for a full layer (head
norm of q, quantised cache write of k and v) against the separate calls it replaces, bit for bit."""
import numpy as np
import pytest

from oracle import oracle as orc
from tests import util

pytestmark = pytest.mark.gpu


def _weights(rng, rows, d_in):
    import torch
    from embla_metal_b200 import attn
    words = rng.integers(0, 2 ** 32, (rows, d_in // 32, 4), dtype=np.uint64).astype(np.uint32)
    sc = orc.to_bits(rng.uniform(0.002, 0.01, (rows, d_in // 64)), orc.BF16)
    bs = orc.to_bits(-7.5 * orc.from_bits(sc, orc.BF16) + rng.standard_normal((rows, d_in // 64)) * 0.002, orc.BF16)   # about -7.5 a: weights centred
    dev = attn.W4Weights(torch.from_numpy(words.view(np.int32)).cuda(), torch.from_numpy(sc.view(np.int16)).cuda(),
                         torch.from_numpy(bs.view(np.int16)).cuda())
    return (words, sc, bs), dev


def _case(batch, Hq, Hkv, dtype, d_in, seed):
    import torch
    from embla_metal_b200 import attn
    rng = np.random.default_rng(seed)
    ctx = attn.Attention(Hq, Hkv, dtype, max_batch=batch, max_context=512)
    host, dev = zip(*[_weights(rng, rows, d_in) for rows in (Hq * 128, Hkv * 128, Hkv * 128)])
    xb = orc.to_bits(rng.standard_normal((batch, d_in)), dtype)
    xt = util.act_tensor(xb, dtype)
    width = (Hq + 2 * Hkv) * 128
    qkv = torch.zeros(batch, width + 64, dtype=xt.dtype, device="cuda")       # (a row stride wider than the row)
    ctx.qkv_project(dev[0], dev[1], dev[2], xt, qkv)
    ctx.check()
    got = util.act_bits(qkv)[:, :width]
    want = np.concatenate([orc.w4_gemv(w, s, b, xb, dtype, nthreads=8) for (w, s, b) in host], axis=1)
    gf, wf = orc.from_bits(got, dtype).astype(np.float64), orc.from_bits(want, dtype).astype(np.float64)
    # one step of the storage dtype, plus what the order of the fp32 sums can move an output that cancels to near zero
    step = (util.BF16_STEP if dtype == orc.BF16 else 2.0 ** -10) * np.abs(wf) + 2e-5
    assert np.all(np.abs(gf - wf) <= step), f"worst {np.abs(gf - wf).max():.3e} over one step of the storage dtype"
    assert (got == want).mean() > 0.98, f"only {(got == want).mean():.4f} of the outputs equal the CPU restatement's bits"
    assert bool((qkv[:, width:] == 0).all())
    return ctx, dev, xt, qkv, rng


@pytest.mark.parametrize("batch", [1, 3, 8, 19, 33, 64])
def test_w4_gemv_against_the_restatement(batch):
    ctx, *_ = _case(batch, 16, 4, orc.F16, 2048, seed=batch)
    ctx.close()


def test_w4_gemv_reference_shape_bf16():
    ctx, *_ = _case(5, 16, 2, orc.BF16, 2048, seed=50)
    ctx.close()
    ctx, *_ = _case(2, 8, 2, orc.BF16, 512, seed=51)
    ctx.close()


@pytest.mark.parametrize("dtype,scale_dtype,norm_k", [(orc.F16, "f16", True), (orc.BF16, "f32", True), (orc.F16, "f16", False)])
def test_fused_epilogue_equals_the_separate_calls(dtype, scale_dtype, norm_k):
    """GEMV -> embla_kv_append -> embla_attn_full_decode with in-kernel head norm, against the fused producer followed by
    embla_attn_full_decode on prenormed queries: the same cache bytes, the same attention output."""
    import torch
    from embla_metal_b200 import attn
    batch, Hq, Hkv, d_in, ctxlen = 5, 16, 4, 2048, 512
    ctx, dev, xt, qkv, rng = _case(batch, Hq, Hkv, dtype, d_in, seed=60 + int(norm_k))
    npg = ctxlen // 128
    sdt = attn.SCALE_F16 if scale_dtype == "f16" else attn.SCALE_F32
    pools = [attn.KVPool(2, Hkv, batch * npg, attn.KV_INT8, sdt) for _ in range(2)]
    fill = torch.randint(0, 256, pools[0].raw().shape, dtype=torch.uint8, device="cuda")
    for pl in pools:
        pl.raw().copy_(fill)
        r = pl.raw().view(-1, pl.raw().shape[-1])
        r[:, 32768:] = 0           # scales of the rows not written here: zero, so that stale codes weigh nothing
    table = torch.arange(batch * npg, dtype=torch.int32, device="cuda").view(batch, npg).contiguous()
    lens = torch.tensor([1, 77, 128, 129, 400], dtype=torch.int32, device="cuda")
    g = tuple(util.act_tensor(orc.to_bits(rng.standard_normal(128) * 0.1, dtype), dtype) for _ in range(2))
    width = Hq * 128
    # separate calls
    k = qkv[:, width:width + Hkv * 128].unsqueeze(1)
    v = qkv[:, width + Hkv * 128:width + 2 * Hkv * 128].unsqueeze(1)
    ctx.kv_append(pools[0], table, 1, lens - 1, k, v, norm_k=norm_k)
    o_a = torch.zeros(batch, width, dtype=qkv.dtype, device="cuda")
    ctx.full_decode(pools[0], table, lens, 1, qkv, o_a, gains=g, max_seq_len=ctxlen)
    # fused producer
    qkv2 = torch.full_like(qkv, 3.0)
    ctx.qkv_project_full_step(dev[0], dev[1], dev[2], xt, qkv2, pools[1], table, lens, 1, gains=g, norm_k=norm_k)
    o_b = torch.zeros_like(o_a)
    ctx.full_decode(pools[1], table, lens, 1, qkv2, o_b, gains=None, max_seq_len=ctxlen)
    ctx.check()
    torch.cuda.synchronize()
    assert torch.equal(pools[0].raw(), pools[1].raw()), "cache bytes differ"
    assert bool((qkv2[:, width:] == 3.0).all()), "the k and v slots of qkv were written"
    assert torch.equal(o_a.view(torch.int16), o_b.view(torch.int16)), "attention outputs differ"
    assert torch.isfinite(o_a.float()).all() and o_a.float().abs().sum() > 0
    for pl in pools:
        pl.close()
    ctx.close()


def test_oproj_into_the_residual_stream():
    """embla_oproj (gemv EPI 3, then EPI 2) on attention-output-like rows against the restatement: x = y, then x += y."""
    import torch
    from embla_metal_b200 import attn
    rng = np.random.default_rng(70)
    batch, Hq, d = 11, 16, 2048
    ctx = attn.Attention(Hq, 4, orc.BF16, max_batch=batch, max_context=256)
    (words, sc, bs), wo = _weights(rng, d, d)
    ob = orc.to_bits(rng.standard_normal((batch, d)) * 0.3, orc.BF16)
    ot = util.act_tensor(ob, orc.BF16)
    x = torch.full((batch, d + 32), 5.0, dtype=torch.float32, device="cuda")
    ctx.oproj(wo, ot, x, accumulate=False)
    ctx.oproj(wo, ot, x, accumulate=True)
    ctx.check()
    y = orc.from_bits(orc.w4_gemv(words, sc, bs, ob, orc.BF16, nthreads=8), orc.BF16).astype(np.float64)
    got = x[:, :d].cpu().numpy().astype(np.float64)
    assert np.all(np.abs(got - 2 * y) <= 2 * (util.BF16_STEP * np.abs(y) + 2e-5))
    assert bool((x[:, d:] == 5.0).all())
    ctx.close()



def test_attention_sublayer_against_the_restatement():
    """x -> q/k/v producer with the fused epilogue -> full-layer decode -> o-projection, against the same chain on the CPU
    restatement (4-bit GEMV, head norm, write_row8 quantisation of the new token, ReLU² attention, 4-bit GEMV), one sequence
    at a time. The GPU's GEMV outputs may sit one storage step from the restatement's, so a code of the new token's row may
    differ by one; everything downstream is compared within the attention tolerance carried through the o-projection."""
    import torch
    from embla_metal_b200 import attn
    rng = np.random.default_rng(80)
    Hq, Hkv, d, dtype = 16, 4, 2048, orc.BF16
    lens = [300, 129]
    batch, ctxlen = len(lens), 384
    ctx = attn.Attention(Hq, Hkv, dtype, max_batch=batch, max_context=ctxlen)
    host, dev = zip(*[_weights(rng, rows, d) for rows in (Hq * 128, Hkv * 128, Hkv * 128)])
    (wo_words, wo_sc, wo_bs), wo = _weights(rng, d, Hq * 128)
    gains = (orc.to_bits(rng.standard_normal(128) * 0.1, dtype), orc.to_bits(rng.standard_normal(128) * 0.1, dtype))
    xb = orc.to_bits(rng.standard_normal((batch, d)), dtype)
    npg = ctxlen // 128
    pool = attn.KVPool(1, Hkv, batch * npg, attn.KV_INT8, attn.SCALE_F32)
    table = torch.arange(batch * npg, dtype=torch.int32, device="cuda").view(batch, npg).contiguous()
    caches = []
    for b, S in enumerate(lens):                      # S - 1 keys already cached; the token at position S - 1 is new
        k, ks, v, vs = util.int8_cache(rng, Hkv, ctxlen, False)
        caches.append((k, ks, v, vs))
        util.fill_pool(pool, 0, table[b].cpu().numpy(), k, ks, v, vs)
    # ---- GPU
    xt = util.act_tensor(xb, dtype)
    qkv = torch.zeros(batch, (Hq + 2 * Hkv) * 128, dtype=xt.dtype, device="cuda")
    lens_t = torch.tensor(lens, dtype=torch.int32, device="cuda")
    gt = tuple(util.act_tensor(x, dtype) for x in gains)
    ctx.qkv_project_full_step(dev[0], dev[1], dev[2], xt, qkv, pool, table, lens_t, 0, gains=gt, norm_k=True)
    o = torch.zeros(batch, Hq * 128, dtype=xt.dtype, device="cuda")
    ctx.full_decode(pool, table, lens_t, 0, qkv, o, gains=None, max_seq_len=ctxlen)
    resid = torch.zeros(batch, d, dtype=torch.float32, device="cuda")
    ctx.oproj(wo, o, resid, accumulate=False)
    ctx.check()
    got = resid.cpu().numpy().astype(np.float64)
    # ---- the restatement
    y = [orc.w4_gemv(w, s, bz, xb, dtype, nthreads=8) for (w, s, bz) in host]          # [batch, rows] bits
    want = np.zeros((batch, d))
    for b, S in enumerate(lens):
        k, ks, v, vs = [a.copy() for a in caches[b]]
        kc, kscale = orc.quantize_rows(y[1][b].reshape(Hkv, 128), dtype, norm=True)
        vc, vscale = orc.quantize_rows(y[2][b].reshape(Hkv, 128), dtype, norm=False)
        k[:, S - 1], ks[:, S - 1], v[:, S - 1], vs[:, S - 1] = kc, kscale, vc, vscale
        ob, _ = orc.full_decode(y[0][b].reshape(Hq, 128), dtype, k, ks, v, vs, S, gains=gains)
        xo = orc.w4_gemv(wo_words, wo_sc, wo_bs, ob.reshape(1, Hq * 128), dtype)
        want[b] = orc.from_bits(xo, dtype)[0]
    err = np.abs(got - want)
    rms = float(np.sqrt((err ** 2).mean() / (want ** 2).mean()))
    assert err.max() <= 2e-2 * max(1.0, np.abs(want).max()) and rms <= 1e-2, f"max-abs {err.max():.3e}, rel-rms {rms:.3e}"
    pool.close()
    ctx.close()


@pytest.mark.parametrize("dtype", [orc.F16, orc.BF16])
def test_fused_sliding_epilogue_equals_the_separate_calls(dtype):
    """GEMV -> ring write (k normed with its gain and rotated) -> sliding attention with the in-kernel norm and RoPE of q,
    against the producer with that work in its epilogue followed by sliding attention on prenormed queries: same ring
    bytes, same attention output."""
    import torch
    from embla_metal_b200 import attn
    batch, Hq, Hkv, d_in = 5, 16, 4, 2048
    ctx, dev, xt, qkv, rng = _case(batch, Hq, Hkv, dtype, d_in, seed=90)
    tdt = torch.bfloat16 if dtype == orc.BF16 else torch.float16
    rings = [attn.Ring(batch, Hkv, 512, 128, tdt) for _ in range(2)]
    fill_k = torch.randn(rings[0].k.shape, device="cuda").to(tdt)
    fill_v = torch.randn(rings[0].v.shape, device="cuda").to(tdt)
    for r in rings:
        r.k.copy_(fill_k)
        r.v.copy_(fill_v)
    lens = torch.tensor([1, 77, 128, 600, 1025], dtype=torch.int32, device="cuda")
    qg = util.act_tensor(orc.to_bits(rng.standard_normal(128) * 0.1, dtype), dtype)
    kg = util.act_tensor(orc.to_bits(rng.standard_normal(128) * 0.1, dtype), dtype)
    width = Hq * 128
    k = qkv[:, width:width + Hkv * 128].unsqueeze(1)
    v = qkv[:, width + Hkv * 128:width + 2 * Hkv * 128].unsqueeze(1)
    ctx.sliding_write(rings[0], lens - 1, k, v, kgain=kg)
    o_a = torch.zeros(batch, width, dtype=qkv.dtype, device="cuda")
    ctx.sliding_decode(rings[0], lens, qkv, o_a, qgain=qg)
    qkv2 = torch.full_like(qkv, 3.0)
    ctx.qkv_project_sliding_step(dev[0], dev[1], dev[2], xt, qkv2, rings[1], lens, qgain=qg, kgain=kg)
    o_b = torch.zeros_like(o_a)
    ctx.sliding_decode(rings[1], lens, qkv2, o_b)
    ctx.check()
    torch.cuda.synchronize()
    assert torch.equal(rings[0].k.view(torch.int16), rings[1].k.view(torch.int16)) and torch.equal(rings[0].v.view(torch.int16), rings[1].v.view(torch.int16)), "ring bytes differ"
    assert bool((qkv2[:, width:] == 3.0).all())
    assert torch.equal(o_a.view(torch.int16), o_b.view(torch.int16)), "attention outputs differ"
    assert torch.isfinite(o_a.float()).all() and o_a.float().abs().sum() > 0
    ctx.close()

