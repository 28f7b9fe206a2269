"""Generates tests/golden/attention_golden.npz: seeded inputs and the CPU oracle's outputs for them.

The reference (Swift + Metal) cannot run where this is built and holds no golden vectors for its
attention path, so these fixtures freeze the oracle's restatement of its kernels: the CPU tests
check the oracle still reproduces them bit for bit, the GPU tests check the CUDA kernels against
them. Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as orc  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "attention_golden.npz")


def build():
    g = {}
    rng = np.random.default_rng(20260101)

    # --- quantised append: bf16 rows, RMS-normed keys, fp32 scales; one all-zero row
    x = (rng.standard_normal((12, 128)) * rng.uniform(0.1, 5.0, (12, 1))).astype(np.float32)
    x[5] = 0.0
    xb = orc.to_bits(x, orc.BF16)
    g["quant_x"] = xb
    g["quant_codes_norm"], g["quant_scales_norm"] = orc.quantize_rows(xb, orc.BF16, norm=True)
    g["quant_codes_plain"], g["quant_scales_plain"] = orc.quantize_rows(xb, orc.BF16, norm=False)
    g["quant_codes_f16s"], g["quant_scales_f16s"] = orc.quantize_rows(orc.to_bits(x, orc.F16), orc.F16, norm=False, scale_f16=True)

    # --- full decode, benchmark shape (16 q / 4 kv heads, fp16, fp16 scales), with scores
    S = 200
    q = orc.to_bits(rng.standard_normal((16, 128)), orc.F16)
    k = rng.integers(-127, 128, (4, S, 128)).astype(np.int8)
    v = rng.integers(-127, 128, (4, S, 128)).astype(np.int8)
    ks = rng.uniform(0.005, 0.02, (4, S)).astype(np.float16).astype(np.float32)
    vs = rng.uniform(0.005, 0.02, (4, S)).astype(np.float16).astype(np.float32)
    o, sc = orc.full_decode(q, orc.F16, k, ks, v, vs, S, want_scores=True)
    g.update(full_q=q, full_k=k, full_v=v, full_ks=ks, full_vs=vs, full_o=o, full_scores=sc)

    # --- full decode, reference shape (2 kv heads, bf16, fp32 scales, fused head norm with gains)
    S = 150
    q = orc.to_bits(rng.standard_normal((16, 128)) * 3.0, orc.BF16)
    g1 = orc.to_bits(rng.standard_normal(128) * 0.1, orc.BF16)
    g2 = orc.to_bits(rng.standard_normal(128) * 0.1, orc.BF16)
    k = rng.integers(-127, 128, (2, S, 128)).astype(np.int8)
    v = rng.integers(-127, 128, (2, S, 128)).astype(np.int8)
    ks = rng.uniform(0.005, 0.02, (2, S)).astype(np.float32)
    vs = rng.uniform(0.005, 0.02, (2, S)).astype(np.float32)
    o, sc = orc.full_decode(q, orc.BF16, k, ks, v, vs, S, gains=(g1, g2), want_scores=True)
    g.update(ref_q=q, ref_g1=g1, ref_g2=g2, ref_k=k, ref_v=v, ref_ks=ks, ref_vs=vs, ref_o=o, ref_scores=sc)

    # --- selection: ties at the threshold, negative values, signed zeros
    S = 1400
    sc = (np.round(rng.standard_normal((2, S)) * 3) / 3).astype(np.float32)
    sc[0, ::7] = -0.0
    sc[1, 5:900] = 0.25
    g["sel_scores"] = sc
    g["sel_idx"] = orc.select_keys(sc, S)

    # --- sparse decode over fp16 keys: short (all keys) and selecting
    for name, S, Hq, Hkv in (("sparse_short", 100, 8, 2), ("sparse_sel", 1160, 4, 1)):
        q = orc.to_bits(rng.standard_normal((Hq, 128)), orc.F16)
        k = rng.standard_normal((Hkv, S, 128)).astype(np.float32)
        k[:, rng.random(S) < 0.02] *= 4.0
        kb, vb = orc.to_bits(k, orc.F16), orc.to_bits(rng.standard_normal((Hkv, S, 128)), orc.F16)
        scores = orc.score_keys(q, orc.F16, kb, S)
        idx = orc.select_keys(scores, S) if S > 1152 else None
        o = orc.sparse_decode(q, orc.F16, kb, None, vb, None, S, idx=idx, kv_kind=1)
        g.update({name + "_q": q, name + "_k": kb, name + "_v": vb, name + "_scores": scores, name + "_o": o})
        if idx is not None:
            g[name + "_idx"] = idx

    # --- sliding: window 128, ring 256, positions crossing the ring boundary, head norm + RoPE with gains (bf16)
    W, RING, T0 = 128, 256, 300
    qg, kg = orc.to_bits(rng.standard_normal(128) * 0.1, orc.BF16), orc.to_bits(rng.standard_normal(128) * 0.1, orc.BF16)
    hk = orc.to_bits(rng.standard_normal((T0, 2, 128)), orc.BF16)
    hv = orc.to_bits(rng.standard_normal((T0, 2, 128)), orc.BF16)
    rk, rv = np.zeros((2, RING, 128), np.uint16), np.zeros((2, RING, 128), np.uint16)
    orc.sliding_write(hk, hv, orc.BF16, rk, rv, 0, kgain=kg)
    q = orc.to_bits(rng.standard_normal((1, 8, 128)), orc.BF16)
    o = orc.sliding_attend(q, orc.BF16, rk, rv, T0 - 1, W, qgain=qg)
    g.update(slide_qg=qg, slide_kg=kg, slide_hist_k=hk, slide_hist_v=hv, slide_ring_k=rk, slide_ring_v=rv, slide_q=q, slide_o=o)

    # --- full prefill chunk: 24 queries appended after 150 cached keys, causal ReLU², bf16 q, fp16 scales
    p0, Tq = 150, 24
    q = orc.to_bits(rng.standard_normal((Tq, 16, 128)), orc.BF16)
    k = rng.integers(-127, 128, (4, p0 + Tq, 128)).astype(np.int8)
    v = rng.integers(-127, 128, (4, p0 + Tq, 128)).astype(np.int8)
    ks = rng.uniform(0.005, 0.02, (4, p0 + Tq)).astype(np.float16).astype(np.float32)
    vs = rng.uniform(0.005, 0.02, (4, p0 + Tq)).astype(np.float16).astype(np.float32)
    o, o32 = orc.full_prefill(q, orc.BF16, k, ks, v, vs, p0, want_f32=True)
    g.update(pre_q=q, pre_k=k, pre_v=v, pre_ks=ks, pre_vs=vs, pre_o=o, pre_o_f32=o32, pre_p0=np.array(p0))
    return g


if __name__ == "__main__":
    np.savez_compressed(OUT, **build())
    print(OUT, os.path.getsize(OUT), "bytes")
