"""GPU parity of the sliding-layer prefill chunk (ring write of the chunk, then windowed softmax attention of
every new token) against the CPU oracle, through the C ABI."""
import numpy as np
import pytest

from oracle import oracle as orc
from tests import util

pytestmark = pytest.mark.gpu


def _case(T, p0, W, RING, Hq, Hkv, dtype, seed, gains=False, rows=None, poison=False, ramp=0.0):
    import torch
    from embla_metal_b200 import attn
    rng = np.random.default_rng(seed)
    ctx = attn.Attention(Hq, Hkv, dtype, 1, RING)
    tdt = torch.bfloat16 if dtype == orc.BF16 else torch.float16
    ring = attn.Ring(1, Hkv, RING, W, tdt)
    qg = kg = None
    if gains:
        qg = orc.to_bits(rng.standard_normal(128) * 0.1, dtype)
        kg = orc.to_bits(rng.standard_normal(128) * 0.1, dtype)
    # slots no token was written to: zeros, or (poison) NaN bit patterns as uninitialised memory may hold
    rk = np.full((Hkv, RING, 128), 0x7FFF if poison else 0, np.uint16)
    rv = np.full((Hkv, RING, 128), 0x7FFF if poison else 0, np.uint16)
    n_hist = min(p0, W)                          # the cached positions the chunk can still see
    if n_hist:
        hk = orc.to_bits(rng.standard_normal((n_hist, Hkv, 128)), dtype)
        hv = orc.to_bits(rng.standard_normal((n_hist, Hkv, 128)), dtype)
        orc.sliding_write(hk, hv, dtype, rk, rv, p0 - n_hist, kgain=kg)
    ring.k.copy_(util.act_tensor(rk[None], dtype))
    ring.v.copy_(util.act_tensor(rv[None], dtype))
    q = orc.to_bits(rng.standard_normal((T, Hq, 128)), dtype)
    # ramp: the keys grow along the chunk, so that a row's maximum keeps rising from block to block by large factors
    k = orc.to_bits(rng.standard_normal((T, Hkv, 128)) * (1.0 + ramp * np.arange(T)[:, None, None] / T), dtype)
    v = orc.to_bits(rng.standard_normal((T, Hkv, 128)), dtype)
    orc.sliding_write(k, v, dtype, rk, rv, p0, kgain=kg)
    want = orc.from_bits(orc.sliding_attend(q, dtype, rk, rv, p0, W, qgain=qg, nthreads=8), dtype)
    pos = torch.tensor([p0], dtype=torch.int32, device="cuda")
    ctx.sliding_write(ring, pos, util.act_tensor(k.reshape(1, T, Hkv * 128), dtype), util.act_tensor(v.reshape(1, T, Hkv * 128), dtype),
                      kgain=None if kg is None else util.act_tensor(kg, dtype))
    qt = util.act_tensor(q.reshape(1, T, Hq * 128), dtype)
    ot = torch.zeros_like(qt)
    attn.sliding_prefill(ctx, ring, pos, qt, ot, qgain=None if qg is None else util.act_tensor(qg, dtype))
    ctx.check()
    got = orc.from_bits(util.act_bits(ot), dtype).reshape(T, Hq, 128)
    step = util.BF16_STEP if dtype == orc.BF16 else 0.0
    ok, msg = util.close(got, want, out_ulp=step, rel_rms=4e-3 if dtype == orc.BF16 else util.REL_RMS)   # bf16: one output step
    assert ok, f"T={T} p0={p0} W={W}: {msg}"
    ctx.close()


def test_config1_sliding_prefill():
    # benchmark configuration 1 (b): 2048-token causal chunk appended after 2048 cached positions, window 1024, ring 4096, fp16, seed 1
    _case(2048, 2048, 1024, 4096, 16, 4, orc.F16, seed=1)


@pytest.mark.parametrize("T,p0", [(1, 0), (2, 0), (3, 5), (130, 0), (257, 1000), (64, 4000)])
def test_sliding_prefill_shapes(T, p0):
    _case(T, p0, 256, 1024, 16, 4, orc.F16, seed=T + p0)


def test_sliding_prefill_reference_shape_norm_rope():
    # the reference's window (128), bf16, fused head norm + RoPE, ring wrap inside the chunk
    _case(300, 3900, 128, 4096, 16, 4, orc.BF16, seed=8, gains=True)
    _case(70, 10, 128, 4096, 8, 1, orc.BF16, seed=9, gains=True)      # 8 query heads on one kv head: one token a CTA


def test_sliding_prefill_tensor_core_path_edges():
    """fp16 chunks of 64 tokens or more over rings of a multiple of 128 slots run on tcgen05: chunk ends inside a block
    with never-written (NaN) slots after it, windows shorter and longer than a block, fused head norm + RoPE, one and
    eight query heads a kv head, a chunk that wraps the ring."""
    _case(130, 0, 256, 1024, 16, 4, orc.F16, seed=11, poison=True)
    _case(200, 70, 100, 1024, 16, 4, orc.F16, seed=12, poison=True)
    _case(333, 900, 1024, 4096, 16, 4, orc.F16, seed=13, gains=True, poison=True)
    _case(96, 5000, 300, 1024, 8, 1, orc.F16, seed=14, gains=True)
    _case(128, 8100, 512, 2048, 4, 4, orc.F16, seed=15)
    # bfloat16 (P = hi + lo): the reference's window and a long one, never-written slots after the chunk
    _case(333, 900, 1024, 4096, 16, 4, orc.BF16, seed=16, gains=True, poison=True)
    _case(2048, 2048, 1024, 4096, 16, 4, orc.BF16, seed=17)


def test_sliding_prefill_rising_maxima():
    """Scores whose maximum grows by many powers of two across the blocks of a window: the kernel's adopted row maximum has
    to move, and O and the row sum with it, several times a row."""
    _case(600, 1000, 512, 2048, 16, 4, orc.F16, seed=18, ramp=8.0)
    _case(600, 1000, 512, 2048, 16, 4, orc.BF16, seed=19, ramp=8.0)
    _case(300, 0, 1024, 4096, 8, 1, orc.F16, seed=20, ramp=5.0)
