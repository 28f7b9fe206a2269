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


def test_probe_every_launch_or_the_first_of_a_step():
    import torch
    from embla_metal_b200 import stack as stk
    st = stk.DecodeStack(stk.cycle_kinds(8), 2, 1536, window=128, ring=512)   # two sparse layers: two scoring launches a step
    st.fill_random(3)
    st.set_positions(1535)
    for first_only, want in ((False, 4), (True, 2)):
        st.set_probe("score", first_only=first_only)
        st.step()
        st.step()
        torch.cuda.synchronize()
        ms, n = st.read_probe()
        assert n == want and ms > 0
    st.close()


def test_step_host_in_groups_of_layers():
    """The host path feeds the query rows in groups of layers on copy streams of their own (embla_stack_decode_layers a
    group): whatever the grouping, the outputs are those of one copy in, one step, one copy out; three steps in a row
    with changing rows check that no group's copy runs ahead of the step before it."""
    import torch
    from embla_metal_b200 import stack as stk
    kinds = stk.cycle_kinds(8) + [stk.FULL, stk.SPARSE_SHARED, stk.SPARSE_SHARED, stk.SLIDING]
    outs = {}
    for group in (0, 4, 3, 1):
        st = stk.DecodeStack(kinds, 3, 2048, window=128, ring=512)
        st.fill_random(2)
        g = torch.Generator().manual_seed(7)
        got = []
        for step in range(3):
            st.set_positions([2000 + step, 1200 + step, 300 + step])
            st.qkv_host.copy_(torch.randn(st.qkv_host.shape, generator=g).to(st.dtype))
            st.step_host(group=group)
            torch.cuda.current_stream().synchronize()
            got.append(st.o_host.clone())
        st.ctx.check()
        outs[group] = got
        st.close()
    for group in (4, 3, 1):
        for a, b in zip(outs[0], outs[group]):
            assert torch.equal(a.view(torch.int16), b.view(torch.int16)), f"groups of {group} layers differ"


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


def test_config4_full_size_step():
    """Benchmark configuration 4 at full size: 64 sequences x 32768 context x 24 layers [sparse, sliding 1024, sliding 1024,
    full int8], seed 4 (a few sequences shorter, one below the selection threshold). The step run twice from the same
    inputs is bit-identical (appends are idempotent, every combine is ordered); for sampled (sequence, layer) pairs the
    step's rows agree with the CPU restatement fed the very pages and rings the step left behind, and the sparse
    layer's selection - recomputed through the single entry points - equals the restatement's bit for bit."""
    import torch
    from oracle import oracle as orc
    from tests import util
    from embla_metal_b200 import attn, stack as stk
    B, CTX, Hq, Hkv = 64, 32768, 16, 4
    st = stk.DecodeStack(stk.cycle_kinds(24), B, CTX, Hq, Hkv, attn.F16, 1024, 4096)
    st.fill_random(seed=4)
    pos = [CTX - 1] * B
    pos[3], pos[7], pos[11] = 20000, 1100, 4095
    st.set_positions(pos)
    g = torch.Generator(device="cuda").manual_seed(104)
    st.qkv.copy_(torch.randn(st.qkv.shape, device="cuda", generator=g).to(st.dtype))
    st.step()
    st.ctx.check()
    first = st.o.clone()
    st.step()
    st.ctx.check()
    assert torch.equal(first.view(torch.int16), st.o.view(torch.int16)), "two steps from the same inputs differ"
    assert torch.isfinite(first.float()).all()
    npg = CTX // 128
    qrow = lambda li, b: st.qkv[li, b, :Hq * 128].view(torch.int16).cpu().numpy().view(np.uint16).reshape(Hq, 128)
    got = lambda li, b: orc.from_bits(first[li, b].view(torch.int16).cpu().numpy().view(np.uint16), orc.F16).reshape(Hq, 128)

    # full layer (layer 3 = slot 0 of the int8 pool) of sequences 5 (32768 keys) and 3 (20001 keys)
    raw = st.full_pool.raw()
    for b in (5, 3):
        S = pos[b] + 1
        pages = raw[st.table[b].long(), 0].cpu().numpy()                      # [npg, Hkv, page_bytes]
        k = pages[:, :, :16384].reshape(npg, Hkv, 128, 128).transpose(1, 0, 2, 3).reshape(Hkv, npg * 128, 128).view(np.int8)
        v = pages[:, :, 16384:32768].reshape(npg, Hkv, 128, 128).transpose(1, 0, 2, 3).reshape(Hkv, npg * 128, 128).view(np.int8)
        sc = np.ascontiguousarray(pages[:, :, 32768:]).view(np.float16).reshape(npg, Hkv, 2, 128).astype(np.float32)
        ks = sc[:, :, 0].transpose(1, 0, 2).reshape(Hkv, npg * 128)
        vs = sc[:, :, 1].transpose(1, 0, 2).reshape(Hkv, npg * 128)
        want = orc.from_bits(orc.full_decode(qrow(3, b), orc.F16, np.ascontiguousarray(k[:, :S]), np.ascontiguousarray(ks[:, :S]),
                                             np.ascontiguousarray(v[:, :S]), np.ascontiguousarray(vs[:, :S]), S)[0], orc.F16)
        ok, msg = util.close(got(3, b), want)
        assert ok, f"full layer, sequence {b}: {msg}"

    # sparse layer (layer 0 = slot 0 of the 16-bit pool) of sequences 5 (selects) and 7 (1101 keys: attends them all)
    raw16 = st.sparse_pool.raw()
    for b in (5, 7):
        S = pos[b] + 1
        n = (S + 127) // 128
        pages = raw16[st.table[b, :n].long(), 0].cpu().numpy().view(np.uint16)   # [n, Hkv, 2 * 128 * 128]
        k = pages[:, :, :16384].reshape(n, Hkv, 128, 128).transpose(1, 0, 2, 3).reshape(Hkv, n * 128, 128)[:, :S]
        v = pages[:, :, 16384:].reshape(n, Hkv, 128, 128).transpose(1, 0, 2, 3).reshape(Hkv, n * 128, 128)[:, :S]
        k, v = np.ascontiguousarray(k), np.ascontiguousarray(v)
        want_idx = None
        if S > 1152:
            want_sc = orc.score_keys(qrow(0, b), orc.F16, k, S, nthreads=8)
            want_idx = orc.select_keys(want_sc, S)
            scores = torch.zeros(1, Hkv, CTX, device="cuda")
            idx = torch.zeros(1, Hkv, 1152, dtype=torch.int32, device="cuda")
            lens = st.seq_lens[b:b + 1]
            st.ctx.score_keys(st.sparse_pool, st.table[b:b + 1], lens, 0, st.qkv[0, b:b + 1, :Hq * 128], scores, max_seq_len=S)
            st.ctx.select_keys(scores, lens, idx, max_seq_len=S)
            st.ctx.check()
            assert np.array_equal(scores[0, :, :S].cpu().numpy().view(np.uint32), want_sc[:, :S].view(np.uint32))
            assert np.array_equal(idx[0].cpu().numpy().view(np.uint32), want_idx), "selection differs"
            assert orc.verify_selection(want_sc, want_idx, S) == 0
        want = orc.from_bits(orc.sparse_decode(qrow(0, b), orc.F16, k, None, v, None, S, idx=want_idx, kv_kind=1), orc.F16)
        ok, msg = util.close(got(0, b), want)
        assert ok, f"sparse layer, sequence {b}: {msg}"

    # sliding layer (layer 1 = ring 0) of sequences 5 and 11 (position 4095: the ring's last slot)
    for b in (5, 11):
        rk = st.rings[0].k[b].view(torch.int16).cpu().numpy().view(np.uint16)
        rv = st.rings[0].v[b].view(torch.int16).cpu().numpy().view(np.uint16)
        want = orc.from_bits(orc.sliding_attend(qrow(1, b)[None], orc.F16, rk, rv, pos[b], 1024), orc.F16)[0]
        ok, msg = util.close(got(1, b), want)
        assert ok, f"sliding layer, sequence {b}: {msg}"
    st.close()


def test_dependent_launch_overlap_changes_nothing():
    """The step's launches overlap through programmatic dependent launch unless EMBLA_NO_PDL=1 is in the environment (read
    once per process): both ways the same inputs give the same bits."""
    import hashlib
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = (
        "import sys, hashlib, torch; sys.path.insert(0, %r)\n"
        "from embla_metal_b200 import stack as stk\n"
        "st = stk.DecodeStack(stk.cycle_kinds(8) + [stk.FULL, stk.SPARSE_SHARED], 6, 4096, window=256, ring=1024)\n"
        "st.fill_random(9); st.set_positions([4095, 3000, 1500, 1151, 1152, 200])\n"
        "g = torch.Generator(device='cuda').manual_seed(1)\n"
        "st.qkv.copy_(torch.randn(st.qkv.shape, device='cuda', generator=g).to(st.dtype))\n"
        "for _ in range(3): st.step()\n"
        "st.ctx.check()\n"
        "print(hashlib.sha256(st.o.view(torch.int16).cpu().numpy().tobytes()).hexdigest())\n" % root)
    digests = []
    # with dependent-launch overlap and cache rows requested ahead of the wait (the default); with the overlap but every
    # request after the wait; with neither
    for no_pdl, no_early in (("0", "0"), ("0", "1"), ("1", "0")):
        env = dict(os.environ, EMBLA_NO_PDL=no_pdl, EMBLA_NO_EARLY=no_early)
        out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=300)
        assert out.returncode == 0, out.stderr[-800:]
        digests.append(out.stdout.strip().splitlines()[-1])
    assert digests[0] == digests[1] == digests[2] and len(digests[0]) == 64


def test_step_replays_from_a_cuda_graph():
    """A whole step (36 kinds of launches with their dependent-launch edges) captured into a CUDA graph on a side stream and
    replayed with other query rows and other positions in the same device arrays gives the bits of the direct calls (the
    second set of positions lies past the first, so that the rows a step appends never land inside what the other step
    reads). Run in a child process, so that a refused capture cannot leave this process's stream in capture mode."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = (
        "import sys, torch; sys.path.insert(0, %r)\n"
        "from embla_metal_b200 import stack as stk\n"
        "st = stk.DecodeStack(stk.cycle_kinds(8) + [stk.FULL, stk.SPARSE_SHARED], 4, 4096, window=256, ring=1024)\n"
        "st.fill_random(4)\n"
        "g = torch.Generator(device='cuda').manual_seed(2)\n"
        "rows = [torch.randn(st.qkv.shape, device='cuda', generator=g).to(st.dtype) for _ in range(2)]\n"
        "poss = [[3000, 1500, 1100, 200], [4095, 3000, 1152, 300]]\n"
        "want = []\n"
        "for r, ps in zip(rows, poss):\n"
        "    st.set_positions(ps); st.max_seq_len = 4096; st.qkv.copy_(r); st.step(); st.ctx.check(); want.append(st.o.clone())\n"
        "graph = torch.cuda.CUDAGraph()\n"
        "with torch.cuda.graph(graph):\n"
        "    st.step()\n"
        "for r, ps, w in zip(rows, poss, want):\n"
        "    st.set_positions(ps); st.qkv.copy_(r); st.o.zero_(); graph.replay(); torch.cuda.synchronize(); st.ctx.check()\n"
        "    assert torch.equal(st.o.view(torch.int16), w.view(torch.int16)), 'replay differs'\n"
        "print('graph ok')\n" % root)
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and "graph ok" in out.stdout, (out.stdout + out.stderr)[-1200:]


def test_prefill_chunk_equals_token_by_token_steps():
    """embla_stack_prefill_chunk (the attention branch of Prefill.encode: per layer the chunk's K/V into the cache, then the
    chunk's attention) against the same tokens fed one at a time through embla_stack_decode_step on a twin stack: the
    caches end bit-identical (int8 pages with their scales, rings) and every token's outputs agree within the attention
    tolerance (the chunk runs the tcgen05 prefill kernels, the steps the decode kernels)."""
    import torch
    from embla_metal_b200 import stack as stk
    from tests import util
    kinds = [stk.SLIDING, stk.FULL, stk.SLIDING, stk.FULL]
    B, T, ctxlen = 2, 150, 1024
    pos0 = [300, 41]
    twins = []
    for _ in range(2):
        st = stk.DecodeStack(kinds, B, ctxlen, window=256, ring=1024)
        st.fill_random(11)
        twins.append(st)
    chunked, stepped = twins
    g = torch.Generator(device="cuda").manual_seed(5)
    qkv = torch.randn(len(kinds), B, T, chunked.qkv_width, device="cuda", generator=g).to(chunked.dtype)
    o = torch.zeros(len(kinds), B, T, chunked.o_width, dtype=chunked.dtype, device="cuda")
    chunked.prefill_chunk(qkv, o, torch.tensor(pos0, dtype=torch.int32, device="cuda"), max_seq_len=max(pos0) + T)
    chunked.ctx.check()
    want = torch.zeros_like(o)
    for t in range(T):
        stepped.set_positions([p + t for p in pos0])
        stepped.qkv.copy_(qkv[:, :, t])
        stepped.step()
        want[:, :, t] = stepped.o
    stepped.ctx.check()
    torch.cuda.synchronize()
    assert torch.equal(chunked.full_pool.raw(), stepped.full_pool.raw()), "int8 caches differ"
    for a, b in zip(chunked.rings, stepped.rings):
        assert torch.equal(a.k, b.k) and torch.equal(a.v, b.v), "rings differ"
    for li in range(len(kinds)):
        ok, msg = util.close(o[li].float().cpu().numpy(), want[li].float().cpu().numpy(), out_ulp=2.0 ** -10)   # one fp16 step
        assert ok, f"layer {li} (kind {kinds[li]}): {msg}"
    # the last layer as the reference's layer 16: its keys and values only
    third = stk.DecodeStack(kinds, B, ctxlen, window=256, ring=1024)
    third.fill_random(11)
    o3 = torch.full_like(o, 3.0)
    third.prefill_chunk(qkv, o3, torch.tensor(pos0, dtype=torch.int32, device="cuda"), kv_only_layers=1, max_seq_len=max(pos0) + T)
    third.ctx.check()
    torch.cuda.synchronize()
    assert torch.equal(third.full_pool.raw(), chunked.full_pool.raw())
    assert torch.equal(o3[:3], o[:3]) and bool((o3[3] == 3.0).all())
    for st in (chunked, stepped, third):
        st.close()


def test_prefill_chunk_refuses_sparse_layers():
    import torch
    from embla_metal_b200 import attn, stack as stk
    st = stk.DecodeStack(stk.cycle_kinds(4), 1, 512, window=128, ring=512)
    qkv = torch.zeros(4, 1, 8, st.qkv_width, dtype=st.dtype, device="cuda")
    o = torch.zeros(4, 1, 8, st.o_width, dtype=st.dtype, device="cuda")
    with pytest.raises(attn.EmblaError) as e:
        st.prefill_chunk(qkv, o, torch.zeros(1, dtype=torch.int32, device="cuda"))
    assert e.value.status == attn.UNSUPPORTED
    st.close()
