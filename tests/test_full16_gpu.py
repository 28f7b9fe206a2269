"""GPU parity of the full layers' ReLU² decode over a 16-bit cache (the reference's build without the int8 cache: attn_full,
Sources/EmblaMetal/Kernels/attention.metal:148-220) against the CPU oracle, through embla_attn_full_decode."""
import numpy as np
import pytest

from oracle import oracle as orc
from tests import util
from tests.test_sparse_sliding_gpu import _pool16

pytestmark = pytest.mark.gpu


def _case(S, Hq, Hkv, dtype, seed, gains=False, scores=False, kscale=1.0):
    import torch
    from embla_metal_b200 import attn
    rng = np.random.default_rng(seed)
    qb = orc.to_bits(rng.standard_normal((Hq, 128)), dtype)
    kb = orc.to_bits(rng.standard_normal((Hkv, S, 128)) * kscale, dtype)
    vb = orc.to_bits(rng.standard_normal((Hkv, S, 128)), dtype)
    g = None
    if gains:
        g = (orc.to_bits(rng.standard_normal(128) * 0.1, dtype), orc.to_bits(rng.standard_normal(128) * 0.1, dtype))
    ctx = attn.Attention(Hq, Hkv, dtype, max_batch=1, max_context=(S + 127) // 128 * 128)
    pool, ids = _pool16(attn, rng, kb, vb, Hkv)
    tbl = torch.from_numpy(ids[None]).cuda()
    lens = torch.tensor([S], dtype=torch.int32, device="cuda")
    qt = util.act_tensor(qb.reshape(1, Hq * 128), dtype)
    ot = torch.zeros_like(qt)
    ldS = (S + 127) // 128 * 128
    sc = torch.full((1, Hkv, ldS), -3.0, device="cuda") if scores else None
    gt = None if g is None else tuple(util.act_tensor(x, dtype) for x in g)
    ctx.full_decode(pool, tbl, lens, 1, qt, ot, gains=gt, scores=sc, max_seq_len=S)
    ctx.check()
    want, want_sc = orc.full_decode(qb, dtype, kb, None, vb, None, S, kv_kind=1, gains=g, want_scores=scores)
    got = orc.from_bits(util.act_bits(ot), dtype).reshape(Hq, 128)
    ok, msg = util.close(got, orc.from_bits(want, dtype), out_ulp=util.BF16_STEP if dtype == orc.BF16 else 2.0 ** -10)
    assert ok, f"S={S} {msg}"
    if scores:
        assert np.array_equal(sc[0, :, :S].cpu().numpy().view(np.uint32), want_sc[:, :S].view(np.uint32)), "scores are not bit-exact"
    ot2 = torch.zeros_like(qt)
    ctx.full_decode(pool, tbl, lens, 1, qt, ot2, gains=gt, max_seq_len=S)
    torch.cuda.synchronize()
    assert torch.equal(ot.view(torch.int16), ot2.view(torch.int16)), "two runs differ"
    pool.close()
    ctx.close()


@pytest.mark.parametrize("S", [1, 2, 63, 64, 65, 127, 129, 1000, 1153, 4096])
def test_full16_lengths(S):
    _case(S, 16, 4, orc.F16, seed=S)


def test_full16_reference_shape_bf16_fused_norm():
    _case(777, 16, 2, orc.BF16, seed=5, gains=True)
    _case(3000, 16, 2, orc.BF16, seed=6, gains=True)


def test_full16_with_scores_and_long_context():
    _case(5000, 16, 4, orc.F16, seed=7, scores=True)
    _case(32768, 16, 4, orc.F16, seed=8)


def test_full16_large_scores():
    # keys eight times the usual size: weights reach the thousands, over fp16's range unless P carries a power of two
    _case(1500, 16, 4, orc.F16, seed=9, kscale=8.0)
    _case(1500, 16, 4, orc.BF16, seed=10, kscale=8.0)


def test_full16_step_refused():
    import torch
    from embla_metal_b200 import attn
    ctx = attn.Attention(16, 4, orc.F16, max_batch=1, max_context=256)
    pool = attn.KVPool(1, 4, 2, attn.KV_16BIT)
    tbl = torch.zeros(1, 2, dtype=torch.int32, device="cuda")
    lens = torch.ones(1, dtype=torch.int32, device="cuda")
    q = torch.zeros(1, 16 * 128, dtype=torch.float16, device="cuda")
    kv = torch.zeros(1, 4 * 128, dtype=torch.float16, device="cuda")
    with pytest.raises(attn.EmblaError) as e:
        ctx.full_step(pool, tbl, lens, 0, q, kv, kv, torch.zeros_like(q))
    assert e.value.status == attn.UNSUPPORTED
    pool.close()
    ctx.close()
