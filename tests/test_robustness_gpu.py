"""Paths that only run when something goes wrong or is moved: a bounded device-side wait that runs out
(made to run out on the host's request: a producer that stops requesting data, never a fault), the
argument checks of the C ABI on a live context, and a cache block copied out of and back into the pool."""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as orc
from tests import util

pytestmark = pytest.mark.gpu
SHORT_WAIT = 200_000          # SM clocks: about a tenth of a millisecond, far beyond any real load


def _full_setup(attn, rng, S_list, Hq=16, Hkv=4, dtype=orc.F16):
    import torch
    B = len(S_list)
    npg = (max(S_list) + 127) // 128
    ctx = attn.Attention(Hq, Hkv, dtype, max_batch=B, max_context=npg * 128)
    pool = attn.KVPool(1, Hkv, B * npg, attn.KV_INT8, attn.SCALE_F16)
    table = rng.permutation(B * npg).reshape(B, npg).astype(np.int32)
    caches = []
    for b, S in enumerate(S_list):
        c = util.int8_cache(rng, Hkv, S, True)
        util.fill_pool(pool, 0, table[b], *c)
        caches.append(c)
    qb = orc.to_bits(rng.standard_normal((B, Hq, 128)), dtype)
    qt = util.act_tensor(qb.reshape(B, Hq * 128), dtype)
    tbl = torch.from_numpy(table).cuda()
    lens = torch.tensor(S_list, dtype=torch.int32, device="cuda")
    return ctx, pool, tbl, lens, qb, qt, caches


@pytest.mark.parametrize("stall_at,scores", [(0, False), (1, False), (0, True)])
def test_full_decode_wait_runs_out_and_context_survives(stall_at, scores):
    """The producer stops at page `stall_at` of every key range: the consumers' wait for it gives up, the kernel
    drains and returns, embla_attn_check reports EMBLA_TIMEOUT, and the next ordinary call is right."""
    import torch
    from embla_metal_b200 import attn
    rng = np.random.default_rng(5 + stall_at)
    S_list = [32 * 1024] if stall_at else [3000, 700]     # long enough for ranges of several pages when stalling later
    ctx, pool, tbl, lens, qb, qt, caches = _full_setup(attn, rng, S_list)
    ot = torch.zeros_like(qt)
    sct = torch.zeros(len(S_list), 4, tbl.shape[1] * 128, device="cuda") if scores else None
    ctx.set_wait_limit(SHORT_WAIT)
    ctx.inject_stall(stall_at)
    ctx.full_decode(pool, tbl, lens, 0, qt, ot, scores=sct, max_seq_len=max(S_list))
    with pytest.raises(attn.EmblaError) as e:
        ctx.check()
    assert e.value.status == attn.TIMEOUT
    ctx.inject_stall(None)
    ctx.set_wait_limit(1 << 30)
    ctx.check()                                            # the error word was cleared
    ctx.full_decode(pool, tbl, lens, 0, qt, ot, scores=sct, max_seq_len=max(S_list))
    ctx.check()
    got = orc.from_bits(util.act_bits(ot), orc.F16).reshape(len(S_list), 16, 128)
    for b, S in enumerate(S_list):
        want, _ = orc.full_decode(qb[b], orc.F16, *caches[b], S)
        ok, msg = util.close(got[b], orc.from_bits(want, orc.F16))
        assert ok, msg
    pool.close()
    ctx.close()


def test_stack_step_wait_runs_out_in_every_streaming_kernel():
    """One decode step of [sparse, sliding, full] past 1152 keys with every producer stalled at its first item:
    the scoring pass, the ring-tile attention and the full-layer attention each give up their waits and return."""
    import torch
    from embla_metal_b200 import attn, stack as stk
    st = stk.DecodeStack([stk.SPARSE, stk.SLIDING, stk.FULL], 2, 2048)
    st.fill_random(seed=3)
    st.set_positions([1500, 1999])
    st.qkv.copy_(torch.randn(st.qkv.shape, device="cuda").to(st.dtype))
    st.step()
    st.ctx.check()
    good = st.o.clone()
    st.set_positions([1500, 1999])
    st.ctx.set_wait_limit(SHORT_WAIT)
    st.ctx.inject_stall(0)
    st.step()
    with pytest.raises(attn.EmblaError) as e:
        st.ctx.check()
    assert e.value.status == attn.TIMEOUT
    st.ctx.inject_stall(None)
    st.ctx.set_wait_limit(1 << 30)
    st.step()      # the same positions again: the appends rewrite the same rows, the result must be the first one's
    st.ctx.check()
    assert torch.equal(st.o.view(torch.int16), good.view(torch.int16))
    st.close()


def test_prefill_wait_runs_out_and_context_survives():
    """The tcgen05 prefill kernel's wind-down: its TMA producer stops at the first side, converters, MMA issuer and
    ReLU² warps give up in turn, TMEM is released, and the next call is right."""
    import torch
    from embla_metal_b200 import attn
    rng = np.random.default_rng(8)
    T, p0, Hq, Hkv, dtype = 200, 333, 16, 4, orc.BF16
    k, ks, v, vs = util.int8_cache(rng, Hkv, p0 + T, True)
    npg = (p0 + T + 127) // 128
    ctx = attn.Attention(Hq, Hkv, dtype, 1, npg * 128)
    pool = attn.KVPool(1, Hkv, npg, attn.KV_INT8, attn.SCALE_F16)
    ids = np.arange(npg, dtype=np.int32)
    util.fill_pool(pool, 0, ids, k, ks, v, vs)
    tbl = torch.from_numpy(ids[None]).cuda()
    qb = orc.to_bits(rng.standard_normal((T, Hq, 128)), dtype)
    qt = util.act_tensor(qb.reshape(1, T, Hq * 128), dtype)
    ot = torch.zeros_like(qt)
    pos0 = torch.tensor([p0], dtype=torch.int32, device="cuda")
    ctx.set_wait_limit(SHORT_WAIT)
    ctx.inject_stall(0)
    attn.full_prefill(ctx, pool, tbl, 0, pos0, qt, ot)
    with pytest.raises(attn.EmblaError) as e:
        ctx.check()
    assert e.value.status == attn.TIMEOUT
    ctx.inject_stall(None)
    ctx.set_wait_limit(1 << 30)
    attn.full_prefill(ctx, pool, tbl, 0, pos0, qt, ot)
    ctx.check()
    got = orc.from_bits(util.act_bits(ot), dtype).reshape(T, Hq, 128)
    _, want = orc.full_prefill(qb, dtype, k, ks, v, vs, p0, nthreads=8, want_f32=True)
    ok, msg = util.close_stored(got, want, util.BF16_STEP)
    assert ok, msg
    pool.close()
    ctx.close()


def test_block_export_import_roundtrip():
    """A block copied out to host memory and into another physical block decodes bit for bit like the original
    (the check of the reference's `embla-bench cache`, Sources/EmblaBenchKit/Cache.swift:60-69, on one block)."""
    import torch
    from embla_metal_b200 import attn
    rng = np.random.default_rng(12)
    S, Hq, Hkv = 700, 16, 4
    npg = (S + 127) // 128
    ctx = attn.Attention(Hq, Hkv, orc.F16, max_batch=2, max_context=npg * 128)
    pool = attn.KVPool(2, Hkv, 2 * npg, attn.KV_INT8, attn.SCALE_F16)
    ids = np.arange(npg, dtype=np.int32)
    for layer in range(2):
        util.fill_pool(pool, layer, ids, *util.int8_cache(rng, Hkv, S, True))
    host = torch.empty(pool.block_bytes, dtype=torch.uint8).pin_memory()
    dev = torch.empty(pool.block_bytes, dtype=torch.uint8, device="cuda")
    for i in range(npg):                       # even blocks through pinned host memory, odd ones device to device
        buf = host if i % 2 == 0 else dev
        pool.export_block(i, buf)
        torch.cuda.synchronize()
        pool.import_block(npg + i, buf)
        torch.cuda.synchronize()
    raw = pool.raw()
    assert torch.equal(raw[:npg], raw[npg:])
    tbl = torch.from_numpy(np.stack([ids, ids + npg])).cuda()
    lens = torch.tensor([S, S], dtype=torch.int32, device="cuda")
    q1 = util.act_tensor(orc.to_bits(rng.standard_normal((1, Hq * 128)), orc.F16), orc.F16)
    qt = q1.repeat(2, 1).contiguous()
    ot = torch.zeros_like(qt)
    ctx.full_decode(pool, tbl, lens, 1, qt, ot, max_seq_len=S)
    ctx.check()
    assert torch.equal(ot[0].view(torch.int16), ot[1].view(torch.int16))
    assert attn.lib().embla_kv_block_export(pool.handle, 2 * npg, C.c_void_p(dev.data_ptr()), None) == attn.BAD_ARG
    pool.close()
    ctx.close()


def test_sliding_decode_without_gain_is_refused():
    """Sliding layers norm q with one gain vector whatever `ng` says: prenormed = 0 without g1 must fail the
    argument check instead of reaching the kernel with a null gain."""
    import torch
    from embla_metal_b200 import attn
    ctx = attn.Attention(16, 4, orc.F16, max_batch=1, max_context=256)
    ring = attn.Ring(1, 4, 256, 128, torch.float16)
    q = torch.zeros(1, 16 * 128, dtype=torch.float16, device="cuda")
    o = torch.zeros_like(q)
    lens = torch.tensor([10], dtype=torch.int32, device="cuda")
    qd = attn.Query(q.data_ptr(), q.stride(0), 0, 0, None, None)
    rc = attn.lib().embla_attn_sliding_decode(ctx.handle, C.byref(ring.desc), C.c_void_p(lens.data_ptr()), 1, C.byref(qd),
                                              C.c_void_p(o.data_ptr()), C.c_int64(o.stride(0)), None)
    assert rc == attn.BAD_ARG and b"gain" in attn.lib().embla_last_error()
    rc = attn.lib().embla_attn_sliding_step(ctx.handle, C.byref(ring.desc), C.c_void_p(lens.data_ptr()), 1, C.byref(qd),
                                            C.c_void_p(q.data_ptr()), C.c_void_p(q.data_ptr()), C.c_int64(q.stride(0)), 1, None,
                                            C.c_void_p(o.data_ptr()), C.c_int64(o.stride(0)), None)
    assert rc == attn.BAD_ARG
    ctx.close()


@pytest.mark.parametrize("S", [65536, 131072])
def test_select_keys_long_rows(S):
    """Rows longer than one CTA holds in registers: a cluster of CTAs per (sequence, kv head) ranks them."""
    import torch
    from embla_metal_b200 import attn
    rng = np.random.default_rng(S)
    Hkv = 2
    ctx = attn.Attention(16, Hkv, orc.F16, max_batch=1, max_context=S)
    scores = rng.standard_normal((1, Hkv, S)).astype(np.float32)
    scores[0, 1] = np.round(scores[0, 1] * 2) / 2          # heavy ties on one head
    st = torch.from_numpy(scores).cuda()
    lens = torch.tensor([S - 5], dtype=torch.int32, device="cuda")
    idx = torch.zeros((1, Hkv, 1152), dtype=torch.int32, device="cuda")
    ctx.select_keys(st, lens, idx, max_seq_len=S)
    ctx.check()
    want = orc.select_keys(scores[0], S - 5)
    assert np.array_equal(idx[0].cpu().numpy().view(np.uint32), want)
    assert orc.verify_selection(scores[0], want, S - 5) == 0
    ctx.close()


def test_prefill_partials_wait_runs_out_and_context_survives(monkeypatch):
    """The one wait of a CTA for other CTAs: the last page range of a prefill unit waits for the partial sums of the ranges
    that announced themselves before it. The diagnostic stall withholds their reports (nothing faults, nothing hangs: the
    ranges finish as always), the wait runs out after the short limit, the counters are left at zero, and the next call is
    right."""
    import torch
    from embla_metal_b200 import attn
    monkeypatch.setenv("EMBLA_PREFILL_BALANCED", "1")   # pieces of a run of pages: every unit's ranges meet in the scratch
    monkeypatch.setenv("EMBLA_PREFILL_REDUCE", "0")     # ... and are added by the unit's last range, not by the kernel behind
    rng = np.random.default_rng(9)
    T, p0, Hq, Hkv, dtype = 200, 6000, 8, 2, orc.BF16
    k, ks, v, vs = util.int8_cache(rng, Hkv, p0 + T, True)
    npg = (p0 + T + 127) // 128
    ctx = attn.Attention(Hq, Hkv, dtype, 1, npg * 128)
    pool = attn.KVPool(1, Hkv, npg, attn.KV_INT8, attn.SCALE_F16)
    ids = np.arange(npg, dtype=np.int32)
    util.fill_pool(pool, 0, ids, k, ks, v, vs)
    tbl = torch.from_numpy(ids[None]).cuda()
    qb = orc.to_bits(rng.standard_normal((T, Hq, 128)), dtype)
    qt = util.act_tensor(qb.reshape(1, T, Hq * 128), dtype)
    ot = torch.zeros_like(qt)
    pos0 = torch.tensor([p0], dtype=torch.int32, device="cuda")
    ctx.set_wait_limit(SHORT_WAIT)
    ctx.inject_stall(attn.Attention.STALL_PARTIALS)
    attn.full_prefill(ctx, pool, tbl, 0, pos0, qt, ot)
    with pytest.raises(attn.EmblaError) as e:
        ctx.check()
    assert e.value.status == attn.TIMEOUT
    ctx.inject_stall(None)
    ctx.set_wait_limit(1 << 30)
    attn.full_prefill(ctx, pool, tbl, 0, pos0, qt, ot)
    ctx.check()
    got = orc.from_bits(util.act_bits(ot), dtype).reshape(T, Hq, 128)
    _, want = orc.full_prefill(qb, dtype, k, ks, v, vs, p0, r0=1, rstep=4, nthreads=8, want_f32=True)
    ok, msg = util.close_stored(got[1::4], want[1::4], util.BF16_STEP)
    assert ok, msg
    pool.close()
    ctx.close()
