"""GPU parity of the tcgen05 prefill-chunk kernel (full layers, causal ReLU² over the int8 cache)
against the CPU oracle, through the C ABI."""
import os

import numpy as np
import pytest

from oracle import oracle as orc
from tests import util

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "attention_golden.npz")


def _prefill(q_bits, k, ks, v, vs, p0, dtype, scale_f16, gains=None, rows=None, nthreads=8, qk8=False):
    """Runs the CUDA kernel on dense caches [Hkv, p0 + T, 128]; returns (got, want) on `rows`: the kernel's stored
    outputs and the oracle's fp32 accumulation (before rounding to the storage dtype)."""
    import torch
    from embla_metal_b200 import attn
    T, Hq = q_bits.shape[0], q_bits.shape[1]
    Hkv, S = k.shape[0], k.shape[1]
    assert S == p0 + T
    npg = (S + 127) // 128
    ctx = attn.Attention(Hq, Hkv, dtype, 1, npg * 128)
    pool = attn.KVPool(2, Hkv, npg + 1, attn.KV_INT8, attn.SCALE_F16 if scale_f16 else attn.SCALE_F32)
    ids = np.random.default_rng(p0 + T).permutation(npg + 1)[:npg].astype(np.int32)
    util.fill_pool(pool, 1, ids, k, ks, v, vs)
    tbl = torch.from_numpy(ids[None]).cuda()
    qt = util.act_tensor(q_bits.reshape(1, T, Hq * 128), dtype)
    ot = torch.zeros_like(qt)
    gt = None if gains is None else tuple(util.act_tensor(x, dtype) for x in gains)
    attn.full_prefill(ctx, pool, tbl, 1, torch.tensor([p0], dtype=torch.int32, device="cuda"), qt, ot, gains=gt, qk8=qk8)
    ctx.check()
    got = orc.from_bits(util.act_bits(ot), dtype).reshape(T, Hq, 128)
    ot2 = torch.zeros_like(qt)
    attn.full_prefill(ctx, pool, tbl, 1, torch.tensor([p0], dtype=torch.int32, device="cuda"), qt, ot2, gains=gt, qk8=qk8)
    torch.cuda.synchronize()
    assert torch.equal(ot.view(torch.int16), ot2.view(torch.int16)), "two runs differ"
    r0, rstep = (0, 1) if rows is None else rows
    _, want = orc.full_prefill(q_bits, dtype, k, ks, v, vs, p0, gains=gains, r0=r0, rstep=rstep, nthreads=nthreads, want_f32=True,
                               qk8=qk8)
    pool.close()
    ctx.close()
    return got[r0::rstep], want[r0::rstep]


def _case(T, p0, Hq, Hkv, dtype, scale_f16, seed, gains=False, rows=None, qk8=False):
    rng = np.random.default_rng(seed)
    q = orc.to_bits(rng.standard_normal((T, Hq, 128)), dtype)
    k, ks, v, vs = util.int8_cache(rng, Hkv, p0 + T, scale_f16)
    g = None
    if gains:
        g = (orc.to_bits(rng.standard_normal(128) * 0.1, dtype), orc.to_bits(rng.standard_normal(128) * 0.1, dtype))
    got, want = _prefill(q, k, ks, v, vs, p0, dtype, scale_f16, gains=g, rows=rows, qk8=qk8)
    ok, msg = util.close_stored(got, want, util.BF16_STEP if dtype == orc.BF16 else 2.0 ** -10)
    assert ok, f"T={T} p0={p0}: {msg}"
    if qk8:
        # how far the int8 queries move the result from the fp32-accumulated attention of the unquantised queries
        # (the reference keeps this build for measurement only): reported, and bounded loosely
        r0, rstep = (0, 1) if rows is None else rows
        _, exact = orc.full_prefill(q, dtype, k, ks, v, vs, p0, gains=g, r0=r0, rstep=rstep, nthreads=8, want_f32=True)
        exact = exact[r0::rstep]
        err = np.abs(got - exact)
        rms = float(np.sqrt((err ** 2).mean() / (exact ** 2).mean()))
        print(f"QK8 T={T} p0={p0}: against unquantised queries max-abs {err.max():.3e}, rel-rms {rms:.3e}")
        assert rms < 3e-2


@pytest.mark.parametrize("T,p0", [(128, 0), (1, 0), (5, 123), (128, 128), (129, 127), (300, 1000), (257, 2047)])
def test_prefill_shapes(T, p0):
    _case(T, p0, 16, 4, orc.BF16, True, seed=T * 7 + p0)


def test_prefill_pages_split_over_ctas():
    # few (tile pair, head) units: each unit's pages are split over several CTAs and the last one adds the partials
    _case(200, 12000, 16, 4, orc.BF16, True, seed=21, rows=(3, 5))
    _case(300, 9000, 8, 2, orc.F16, True, seed=22, rows=(0, 7))


def test_prefill_reference_shape_gains_fp32_scales():
    _case(200, 333, 16, 2, orc.BF16, False, seed=3, gains=True)


def test_prefill_fp16_activations():
    _case(140, 77, 16, 4, orc.F16, True, seed=5)


@pytest.mark.parametrize("T,p0", [(128, 0), (5, 123), (300, 1000), (257, 2047)])
def test_prefill_qk8_shapes(T, p0):
    """The int8 Q Kᵀ build against the restatement of the reference's QK8 arithmetic (integer dots are exact on both sides)."""
    _case(T, p0, 16, 4, orc.BF16, True, seed=T * 11 + p0, qk8=True)


def test_prefill_qk8_reference_shape_and_fp16():
    _case(200, 333, 16, 2, orc.BF16, False, seed=4, gains=True, qk8=True)
    _case(140, 77, 16, 4, orc.F16, True, seed=6, qk8=True)
    _case(200, 12000, 16, 4, orc.BF16, True, seed=23, rows=(3, 5), qk8=True)      # pages split over CTAs


def test_prefill_qk8_config3_size():
    _case(2048, 30720, 16, 4, orc.BF16, True, seed=3, rows=(5, 37), qk8=True)


def test_prefill_golden():
    g = np.load(GOLD)
    got, _ = _prefill(g["pre_q"], g["pre_k"], g["pre_ks"], g["pre_v"], g["pre_vs"], int(g["pre_p0"]), orc.BF16, True)
    ok, msg = util.close_stored(got, g["pre_o_f32"], util.BF16_STEP)
    assert ok, msg


def test_config3_prefill_2048_after_30720():
    # benchmark configuration 3: 2048-token chunk after 30720 cached positions, bf16 q, int8 KV + fp16 scales, seed 3.
    # The oracle checks every 37th query row (the full 0.5 TFLOP on the CPU would take minutes).
    _case(2048, 30720, 16, 4, orc.BF16, True, seed=3, rows=(5, 37))


@pytest.fixture
def balanced_launch():
    """The launcher reads EMBLA_PREFILL_BALANCED at every call: 1 takes the balanced launch (one run of pages an SM, cut
    where units end, pieces longest first) wherever it fits instead of where it is estimated to be faster."""
    old = os.environ.get("EMBLA_PREFILL_BALANCED")
    os.environ["EMBLA_PREFILL_BALANCED"] = "1"
    yield
    if old is None:
        del os.environ["EMBLA_PREFILL_BALANCED"]
    else:
        os.environ["EMBLA_PREFILL_BALANCED"] = old


@pytest.mark.parametrize("T,p0,Hq,Hkv", [(300, 9000, 8, 2), (257, 2047, 16, 4), (600, 20000, 16, 4), (128, 128, 16, 4), (5, 123, 16, 2)])
def test_prefill_balanced_launch(balanced_launch, T, p0, Hq, Hkv):
    # units of different lengths cut into pieces: few long units (pieces of many CTAs meet in one unit), many short ones
    # (runs shorter than a unit's tile pair), and chunks so short that some runs hold a page or none
    _case(T, p0, Hq, Hkv, orc.BF16, True, seed=T + p0, rows=(1, 3))


def test_prefill_balanced_launch_qk8_fp16(balanced_launch):
    _case(300, 9000, 8, 2, orc.F16, True, seed=31, rows=(0, 7), qk8=True)
    _case(200, 333, 16, 2, orc.BF16, False, seed=32, gains=True)


def test_prefill_balanced_launch_two_sequences(balanced_launch):
    """Two sequences at different positions in one call: the units of both lie end to end in the piece table. A unit's
    pieces are added in range order whichever CTA finishes last, so two runs agree bit for bit."""
    import torch
    from embla_metal_b200 import attn
    rng = np.random.default_rng(77)
    T, Hq, Hkv, p0s = 260, 8, 2, [5000, 1300]
    caches = [util.int8_cache(rng, Hkv, p0 + T, True) for p0 in p0s]
    qs = [orc.to_bits(rng.standard_normal((T, Hq, 128)), orc.BF16) for _ in p0s]
    npgs = [(p0 + T + 127) // 128 for p0 in p0s]
    ctx = attn.Attention(Hq, Hkv, orc.BF16, 2, max(npgs) * 128)
    pool = attn.KVPool(1, Hkv, sum(npgs), attn.KV_INT8, attn.SCALE_F16)
    ids = rng.permutation(sum(npgs)).astype(np.int32)
    tbl = np.zeros((2, max(npgs)), dtype=np.int32)
    at = 0
    for b, (k, ks, v, vs) in enumerate(caches):
        tbl[b, :npgs[b]] = ids[at:at + npgs[b]]
        util.fill_pool(pool, 0, tbl[b, :npgs[b]], k, ks, v, vs)
        at += npgs[b]
    tblt = torch.from_numpy(tbl).cuda()
    qt = util.act_tensor(np.stack([q.reshape(T, Hq * 128) for q in qs]), orc.BF16)
    pos = torch.tensor(p0s, dtype=torch.int32, device="cuda")
    both, again = torch.zeros_like(qt), torch.zeros_like(qt)
    attn.full_prefill(ctx, pool, tblt, 0, pos, qt, both)
    attn.full_prefill(ctx, pool, tblt, 0, pos, qt, again)
    ctx.check()
    assert torch.equal(both.view(torch.int16), again.view(torch.int16)), "two runs differ"
    for b in range(2):
        got = orc.from_bits(util.act_bits(both[b]), orc.BF16).reshape(T, Hq, 128)
        k, ks, v, vs = caches[b]
        _, want = orc.full_prefill(qs[b], orc.BF16, k, ks, v, vs, p0s[b], r0=2, rstep=5, nthreads=8, want_f32=True)
        ok, msg = util.close_stored(got[2::5], want[2::5], util.BF16_STEP)
        assert ok, f"sequence {b}: {msg}"
    pool.close()
    ctx.close()


@pytest.mark.parametrize("balanced,reduce", [("0", "1"), ("0", "0"), ("1", "1"), ("1", "0")])
def test_prefill_ranges_through_scratch_both_ways(monkeypatch, balanced, reduce):
    """Page ranges that meet in the scratch, as an even split of every unit (balanced 0: clusters off, so the split goes
    through the scratch) or as pieces of the balanced launch, added by the unit's last range (reduce 0) or by the kernel
    launched behind (reduce 1)."""
    monkeypatch.setenv("EMBLA_PREFILL_BALANCED", balanced)
    monkeypatch.setenv("EMBLA_PREFILL_REDUCE", reduce)
    monkeypatch.setenv("EMBLA_NO_CLUSTER", "1")
    _case(200, 12000, 16, 4, orc.BF16, True, seed=41, rows=(3, 5))
    _case(300, 9000, 8, 2, orc.F16, True, seed=42, rows=(0, 7))
    _case(257, 4000, 16, 2, orc.BF16, False, seed=43, gains=True, rows=(2, 9), qk8=True)
