"""The native decode step (embla_stack_decode_step) over small stacks of every layer kind against the single-kernel
entry points it is made of — including the reference's block structure: a full layer that scores keys, the selection,
and sparse layers over the same int8 cache."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_reference_block_through_the_stack():
    import torch
    from embla_metal_b200 import attn, stack as stk
    ctxlen, B = 2048, 3
    kinds = [stk.SLIDING, stk.FULL, stk.SPARSE_SHARED, stk.SPARSE_SHARED, stk.SPARSE]
    st = stk.DecodeStack(kinds, B, ctxlen, window=256, ring=1024)
    st.fill_random(5)
    st.set_positions([ctxlen - 1, 1500, 700])           # two sequences select, one attends every key
    st.qkv.copy_(torch.randn(st.qkv.shape, device="cuda").to(st.dtype))
    st.step()
    st.ctx.check()
    got = st.o.clone()
    assert torch.isfinite(got.float()).all()
    # the same through the single entry points (the full layer's append has already happened: appends are idempotent)
    Hq, Hkv = st.Hq, st.Hkv
    q = lambda li: st.qkv[li][:, :Hq * 128]
    o = torch.zeros_like(st.o[0])
    scores = torch.zeros(B, Hkv, ctxlen, device="cuda")
    idx = torch.zeros(B, Hkv, 1152, dtype=torch.int32, device="cuda")
    st.ctx.full_decode(st.full_pool, st.table, st.seq_lens, 0, q(1), o, scores=scores, max_seq_len=st.max_seq_len)
    assert torch.equal(o, got[1])
    st.ctx.select_keys(scores, st.seq_lens, idx, max_seq_len=st.max_seq_len)
    import ctypes as C
    for li in (2, 3):
        view = attn.Attention.view(st.table, st.seq_lens, 0, st.max_seq_len)
        qd = attn.Attention.query(q(li), None)
        attn._check(attn.lib().embla_attn_sparse_decode_int8(st.ctx.handle, st.full_pool.handle, C.byref(view), C.byref(qd),
                                                             C.c_void_p(idx.data_ptr()), C.c_void_p(o.data_ptr()),
                                                             C.c_int64(o.stride(0)), attn._stream()))
        assert torch.equal(o, got[li])
    # the sparse layer with its own 16-bit keys: score -> select -> attend
    st.ctx.score_keys(st.sparse_pool, st.table, st.seq_lens, 0, q(4), scores, max_seq_len=st.max_seq_len)
    st.ctx.select_keys(scores, st.seq_lens, idx, max_seq_len=st.max_seq_len)
    st.ctx.sparse_decode(st.sparse_pool, st.table, st.seq_lens, 0, q(4), o, idx=idx, max_seq_len=st.max_seq_len)
    assert torch.equal(o, got[4])
    st.ctx.sliding_decode(st.rings[0], st.seq_lens, q(0), o)
    assert torch.equal(o, got[0])
    assert st.launches_per_step() == 1 + 2 + 1 + 1 + 3   # sliding; full (append fused) + select; shared x 2; score (append fused) + select + attend
    st.close()


def test_step_host_round_trip_and_probe():
    import torch
    from embla_metal_b200 import stack as stk
    st = stk.DecodeStack(stk.cycle_kinds(4), 2, 1536, window=128, ring=512)
    st.fill_random(1)
    st.set_positions(1535)
    st.qkv_host.copy_(torch.randn(st.qkv_host.shape).to(st.dtype))
    st.set_probe("score")
    st.step_host()
    torch.cuda.synchronize()
    ms, n = st.read_probe()
    assert n == 1 and ms > 0
    a = st.o_host.clone()
    st.set_probe(None)
    st.step_host()
    torch.cuda.synchronize()
    assert torch.equal(a, st.o_host)          # same inputs, same position: bit-identical (appends are idempotent)
    assert torch.isfinite(a.float()).all() and a.float().abs().sum() > 0
    st.close()


def test_fused_sliding_step_equals_write_then_attend():
    """embla_attn_sliding_step (ring write + attention in one launch, the reference's attn_sliding) against
    embla_sliding_write followed by embla_attn_sliding_decode: same ring contents, same outputs, bit for bit."""
    import ctypes as C
    import torch
    from embla_metal_b200 import attn
    torch.manual_seed(3)
    B, Hq, Hkv, RING, W = 5, 16, 4, 1024, 256
    for dtype, tdt in ((attn.F16, torch.float16), (attn.BF16, torch.bfloat16)):
        ctx = attn.Attention(Hq, Hkv, dtype, B, RING)
        r1, r2 = attn.Ring(B, Hkv, RING, W, tdt), attn.Ring(B, Hkv, RING, W, tdt)
        hist = torch.randn(r1.k.shape, device="cuda").to(tdt)
        r1.k.copy_(hist); r2.k.copy_(hist)
        hv = torch.randn(r1.v.shape, device="cuda").to(tdt)
        r1.v.copy_(hv); r2.v.copy_(hv)
        pos = torch.tensor([0, 5, 255, 1023, 3000], dtype=torch.int32, device="cuda")
        lens = pos + 1
        q = torch.randn(B, Hq * 128, device="cuda").to(tdt)
        k = torch.randn(B, 1, Hkv * 128, device="cuda").to(tdt)
        v = torch.randn(B, 1, Hkv * 128, device="cuda").to(tdt)
        qg = (torch.randn(128, device="cuda") * 0.1).to(tdt)
        kg = (torch.randn(128, device="cuda") * 0.1).to(tdt)
        o1, o2 = torch.zeros_like(q), torch.zeros_like(q)
        ctx.sliding_write(r1, pos, k, v, kgain=kg)
        ctx.sliding_decode(r1, lens, q, o1, qgain=qg)
        qd = attn.Attention.query(q, (qg, None))
        attn._check(attn.lib().embla_attn_sliding_step(ctx.handle, C.byref(r2.desc), C.c_void_p(lens.data_ptr()), B, C.byref(qd),
                                                       C.c_void_p(k.data_ptr()), C.c_void_p(v.data_ptr()), C.c_int64(k.stride(0)), 0,
                                                       C.c_void_p(kg.data_ptr()), C.c_void_p(o2.data_ptr()), C.c_int64(o2.stride(0)),
                                                       attn._stream()))
        ctx.check()
        assert torch.equal(r1.k.view(torch.int16), r2.k.view(torch.int16)) and torch.equal(r1.v.view(torch.int16), r2.v.view(torch.int16))
        assert torch.equal(o1.view(torch.int16), o2.view(torch.int16))
        ctx.close()
