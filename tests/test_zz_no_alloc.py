"""The allocation-free full-layer decode entry point against the regular one, through the C ABI.

Hosts that have handed all device memory to their own arena, or that run attention on a thread where
cudaMalloc is forbidden, call embla_attn_full_decode_noalloc: it needs no context object and keeps
its split-K scratch in a fixed array inside the library. This file is collected last on purpose, so
that a run stopping at the first failure has already run every other test. The check is done twice in
a row because every call reuses the same array (stale partial sums or counters from the first call
must not leak into the second).
"""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as orc
from tests import util

pytestmark = pytest.mark.gpu


def _noalloc(attn, pool, tbl, lens, layer, q, o, n_q_heads, act_dtype, max_seq_len, gains=None):
    import torch
    view = attn.Attention.view(tbl, lens, layer, max_seq_len)
    qd = attn.Attention.query(q, gains)
    fn = attn.lib().embla_attn_full_decode_noalloc
    return fn(pool.handle, C.byref(view), C.byref(qd), n_q_heads, act_dtype, C.c_void_p(o.data_ptr()),
              C.c_int64(o.stride(0)), C.c_void_p(torch.cuda.current_stream().cuda_stream))


@pytest.mark.parametrize("Hkv,dtype,scale_f16,gains", [(4, orc.F16, True, False), (2, orc.BF16, False, True)])
def test_noalloc_matches_oracle_and_regular_twice(Hkv, dtype, scale_f16, gains):
    """Against the CPU oracle (tolerance of every attention test) and, bit for bit, against the entry point that takes a
    context: both run the same kernel with the same key split. The second shape is the reference's own: 8 query heads a
    kv head (the widest partial rows of the fixed array), bf16, fp32 scales, head norm fused."""
    import torch
    from embla_metal_b200 import attn
    rng = np.random.default_rng(77 + Hkv)
    Hq = 16
    S_list = [3000, 257, 1, 4096]
    B, npg = len(S_list), 32
    ctx = attn.Attention(Hq, Hkv, dtype, max_batch=B, max_context=npg * 128)
    pool = attn.KVPool(1, Hkv, B * npg, attn.KV_INT8, attn.SCALE_F16 if scale_f16 else attn.SCALE_F32)
    table = rng.permutation(B * npg).reshape(B, npg).astype(np.int32)
    caches = [util.int8_cache(rng, Hkv, S, scale_f16) for S in S_list]
    for b in range(B):
        util.fill_pool(pool, 0, table[b], *caches[b])
    tbl = torch.from_numpy(table).cuda()
    lens = torch.tensor(S_list, dtype=torch.int32, device="cuda")
    g = gt = None
    if gains:
        g = (orc.to_bits(rng.standard_normal(128) * 0.1, dtype), orc.to_bits(rng.standard_normal(128) * 0.1, dtype))
        gt = tuple(util.act_tensor(x, dtype) for x in g)
    for call in range(2):
        qb = orc.to_bits(rng.standard_normal((B, Hq, 128)), dtype)
        q = util.act_tensor(qb.reshape(B, Hq * 128), dtype)
        same = torch.zeros_like(q)
        ctx.full_decode(pool, tbl, lens, 0, q, same, gains=gt, max_seq_len=max(S_list))
        got = torch.full_like(q, 7.0)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        status = _noalloc(attn, pool, tbl, lens, 0, q, got, Hq, dtype, max(S_list), gains=gt)
        assert status == attn.OK, attn.lib().embla_last_error().decode()
        torch.cuda.synchronize()
        # what the entry point is for: once a device's set-up call is done, a call takes no device memory
        if call > 0:
            assert torch.cuda.mem_get_info()[0] == free_before, "a call after the first changed the free device memory"
        assert torch.equal(got.view(torch.int16), same.view(torch.int16)), f"call {call}: differs from embla_attn_full_decode"
        got_f = orc.from_bits(util.act_bits(got), dtype).reshape(B, Hq, 128)
        for b, S in enumerate(S_list):
            want, _ = orc.full_decode(qb[b], dtype, *caches[b], S, gains=g)
            ok, msg = util.close(got_f[b], orc.from_bits(want, dtype), out_ulp=util.BF16_STEP if dtype == orc.BF16 else 0.0)
            assert ok, f"call {call}, sequence {b}: {msg}"
    pool.close()
    ctx.close()


def test_noalloc_rejects_oversize_batch():
    import torch
    from embla_metal_b200 import attn
    Hq, Hkv = 16, 4
    pool = attn.KVPool(1, Hkv, 2, attn.KV_INT8, attn.SCALE_F16)
    B = 65   # 65 x 4 kv heads = 260 pairs, over the fixed scratch's 256
    tbl = torch.zeros((B, 1), dtype=torch.int32, device="cuda")
    lens = torch.ones(B, dtype=torch.int32, device="cuda")
    q = torch.zeros((B, Hq * 128), dtype=torch.float16, device="cuda")
    o = torch.zeros_like(q)
    status = _noalloc(attn, pool, tbl, lens, 0, q, o, Hq, orc.F16, 128)
    assert status == attn.BAD_ARG
    assert "256" in attn.lib().embla_last_error().decode()
    pool.close()
