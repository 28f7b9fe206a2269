"""Shared helpers of the tests: seeded inputs in the shapes of the benchmark configurations, pool
filling, and the tolerance check (2e-3 max-abs and 1e-3 relative RMS against the fp32 oracle)."""
import numpy as np

from oracle import oracle as orc

MAX_ABS, REL_RMS = 2e-3, 1e-3


def close(got, want, max_abs=MAX_ABS, rel_rms=REL_RMS, out_ulp=0.0):
    """Both arrays are already rounded to the 16-bit output dtype. `out_ulp` = that dtype's relative step
    (2^-7 for bfloat16): two fp32 results that agree to 1e-6 can still round to neighbouring bf16 values,
    so one output step is allowed on top of the fp32 tolerance where outputs are large."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    excess = (np.abs(got - want) - out_ulp * np.abs(want)).max()
    err = np.abs(got - want).max()
    rms = np.sqrt(((got - want) ** 2).mean() / max((want ** 2).mean(), 1e-30))
    return excess <= max_abs and rms <= rel_rms, f"max-abs {err:.3e} (<= {max_abs} + {out_ulp:.1e}|x|), rel-rms {rms:.3e} (<= {rel_rms})"


BF16_STEP = 2.0 ** -7


def close_stored(got, want_f32, out_step, max_abs=MAX_ABS, rel_rms=REL_RMS):
    """`got` is a kernel's output after rounding to its 16-bit storage dtype, `want_f32` the oracle's fp32
    accumulation before that rounding. Storing rounds by up to half a step (out_step * |x| bounds one step),
    which is not the kernel's error: only what exceeds half a step is held against the fp32 tolerances."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want_f32, np.float64)
    err = np.maximum(np.abs(got - want) - 0.5 * out_step * np.abs(want), 0.0)
    rms = np.sqrt((err ** 2).mean() / max((want ** 2).mean(), 1e-30))
    return err.max() <= max_abs and rms <= rel_rms, (f"beyond storage rounding: max-abs {err.max():.3e} (<= {max_abs}), "
                                                     f"rel-rms {rms:.3e} (<= {rel_rms})")


def int8_cache(rng, Hkv, S, scale_f16=True, lo=0.005, hi=0.02):
    """K/V int8 uniform in [-127, 127] with per-token per-head scales uniform in [lo, hi]."""
    k = rng.integers(-127, 128, (Hkv, S, 128)).astype(np.int8)
    v = rng.integers(-127, 128, (Hkv, S, 128)).astype(np.int8)
    ks = rng.uniform(lo, hi, (Hkv, S)).astype(np.float32)
    vs = rng.uniform(lo, hi, (Hkv, S)).astype(np.float32)
    if scale_f16:
        ks = ks.astype(np.float16).astype(np.float32)
        vs = vs.astype(np.float16).astype(np.float32)
    return k, ks, v, vs


def page_bytes_np(k, ks, v, vs, scale_f16):
    """int8 pages [Hkv, npages, page_bytes] (uint8) of dense caches [Hkv, S, 128], zero padded."""
    Hkv, S = k.shape[0], k.shape[1]
    npg = (S + 127) // 128
    sdt = np.float16 if scale_f16 else np.float32
    ssz = 2 if scale_f16 else 4
    pages = np.zeros((Hkv, npg, 32768 + 256 * ssz), np.uint8)

    def pad(a, shape):
        out = np.zeros(shape, a.dtype)
        out[tuple(slice(0, n) for n in a.shape)] = a
        return out

    kp = pad(k, (Hkv, npg * 128, 128)).reshape(Hkv, npg, 128 * 128).view(np.uint8)
    vp = pad(v, (Hkv, npg * 128, 128)).reshape(Hkv, npg, 128 * 128).view(np.uint8)
    ksp = pad(ks.astype(sdt), (Hkv, npg * 128)).reshape(Hkv, npg, 128).view(np.uint8)
    vsp = pad(vs.astype(sdt), (Hkv, npg * 128)).reshape(Hkv, npg, 128).view(np.uint8)
    pages[:, :, :16384] = kp
    pages[:, :, 16384:32768] = vp
    pages[:, :, 32768:32768 + 128 * ssz] = ksp
    pages[:, :, 32768 + 128 * ssz:] = vsp
    return pages


def fill_pool(pool, layer, blocks, k, ks, v, vs):
    """Writes dense int8 caches of one sequence into `pool` at physical blocks `blocks` (list)."""
    import torch
    from embla_metal_b200 import attn
    pages = page_bytes_np(k, ks, v, vs, pool.scale_dtype == attn.SCALE_F16)
    raw = pool.raw()
    t = torch.from_numpy(pages).cuda()
    idx = torch.as_tensor(list(blocks[:pages.shape[1]]), device="cuda", dtype=torch.long)
    raw[idx, layer] = t.permute(1, 0, 2)


def act_tensor(bits, dtype):
    """uint16 numpy storage -> torch tensor of the activation dtype on the GPU."""
    import torch
    t = torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).cuda()
    return t.view(torch.bfloat16 if dtype == orc.BF16 else torch.float16)


def act_bits(t):
    """torch 16-bit tensor -> uint16 numpy storage."""
    import torch
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def stack_oracle_rows(st, li, b, pos_b):
    """What the CPU oracle gives for layer `li`, sequence `b` of a DecodeStack after a step at position `pos_b`, fed the
    very pages and rings the step left behind and the step's query row (fp16 stacks, queries prenormed). Returns
    [Hq, 128] floats; for a sparse layer past 1152 keys the oracle scores and selects the keys itself."""
    import torch
    from embla_metal_b200 import stack as stk
    Hq, Hkv, S = st.Hq, st.Hkv, pos_b + 1
    kind = st.kinds[li]
    q = st.qkv[li, b, :Hq * 128].view(torch.int16).cpu().numpy().view(np.uint16).reshape(Hq, 128)
    slot = sum(1 for k in st.kinds[:li] if k == kind)
    n = (S + 127) // 128
    if kind == stk.FULL:
        pages = st.full_pool.raw()[st.table[b, :n].long(), slot].cpu().numpy()        # [n, Hkv, page_bytes]
        k = pages[:, :, :16384].reshape(n, Hkv, 128, 128).transpose(1, 0, 2, 3).reshape(Hkv, n * 128, 128).view(np.int8)
        v = pages[:, :, 16384:32768].reshape(n, Hkv, 128, 128).transpose(1, 0, 2, 3).reshape(Hkv, n * 128, 128).view(np.int8)
        sc = np.ascontiguousarray(pages[:, :, 32768:]).view(np.float16).reshape(n, Hkv, 2, 128).astype(np.float32)
        ks = sc[:, :, 0].transpose(1, 0, 2).reshape(Hkv, n * 128)
        vs = sc[:, :, 1].transpose(1, 0, 2).reshape(Hkv, n * 128)
        c = np.ascontiguousarray
        return orc.from_bits(orc.full_decode(q, orc.F16, c(k[:, :S]), c(ks[:, :S]), c(v[:, :S]), c(vs[:, :S]), S)[0], orc.F16)
    if kind == stk.SPARSE:
        pages = st.sparse_pool.raw()[st.table[b, :n].long(), slot].cpu().numpy().view(np.uint16)   # [n, Hkv, 2 * 128 * 128]
        k = np.ascontiguousarray(pages[:, :, :16384].reshape(n, Hkv, 128, 128).transpose(1, 0, 2, 3).reshape(Hkv, n * 128, 128)[:, :S])
        v = np.ascontiguousarray(pages[:, :, 16384:].reshape(n, Hkv, 128, 128).transpose(1, 0, 2, 3).reshape(Hkv, n * 128, 128)[:, :S])
        idx = orc.select_keys(orc.score_keys(q, orc.F16, k, S, nthreads=4), S) if S > 1152 else None
        return orc.from_bits(orc.sparse_decode(q, orc.F16, k, None, v, None, S, idx=idx, kv_kind=1), orc.F16)
    if kind == stk.SLIDING:
        ring = st.rings[slot]
        rk = ring.k[b].view(torch.int16).cpu().numpy().view(np.uint16)
        rv = ring.v[b].view(torch.int16).cpu().numpy().view(np.uint16)
        window = ring.desc.window
        return orc.from_bits(orc.sliding_attend(q[None], orc.F16, rk, rv, pos_b, window), orc.F16)[0]
    raise ValueError(f"layer kind {kind}")
