"""The CPU oracle against independent float64 numpy formulas, against properties of the domain, and
against the committed golden fixtures (which freeze its behaviour). No GPU."""
import os

import numpy as np
import pytest

from oracle import oracle as orc
from tests import util

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "attention_golden.npz")


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLD)


def _f(bits, dtype):
    return orc.from_bits(bits, dtype).astype(np.float64)


def _head_norm64(x, gains, dtype):
    r = 1.0 / np.sqrt((x ** 2).mean(-1, keepdims=True) + 1.1920929e-07)
    g = 1.0
    for w in gains:
        g = g * (1.0 + _f(w, dtype))
    return x * r * g


def _rope64(x, pos):
    x = x.copy()
    l = np.arange(32)
    theta = -pos * 2.0 ** (-l / 32.0 * 13.287712379549449)
    c, s = np.cos(theta), np.sin(theta)
    x1, x2 = x[..., :32].copy(), x[..., 32:64].copy()
    x[..., :32] = x1 * c - x2 * s
    x[..., 32:64] = x1 * s + x2 * c
    return x


def _relu2_64(q, k, ks, v, vs, G):
    out = np.zeros((q.shape[0], 128))
    for h in range(q.shape[0]):
        kvh = h // G
        t = (k[kvh].astype(np.float64) @ q[h]) * ks[kvh]
        w = np.maximum(t / np.sqrt(128.0), 0.0) ** 2
        out[h] = (w * vs[kvh]) @ v[kvh].astype(np.float64) / (np.sqrt(128.0) + w.sum())
    return out


def test_config0_full_decode_vs_float64():
    # benchmark configuration 0: 16 q / 4 kv heads, context 1024, fp16 q ~ N(0,1), int8 K/V, fp16 scales in [0.005, 0.02], seed 0
    rng = np.random.default_rng(0)
    q = orc.to_bits(rng.standard_normal((16, 128)), orc.F16)
    k, ks, v, vs = util.int8_cache(rng, 4, 1024, True)
    o, sc = orc.full_decode(q, orc.F16, k, ks, v, vs, 1024, want_scores=True)
    want = _relu2_64(_f(q, orc.F16), k, ks, v, vs, 4)
    ok, msg = util.close(orc.from_bits(o, orc.F16), want)
    assert ok, msg
    # scores: max over the kv head's 4 query heads of q.k * kscale, no 1/sqrt(D)
    t = np.einsum("hd,gsd->hgs", _f(q, orc.F16), k.astype(np.float64))
    want_sc = np.stack([(t[4 * g:4 * g + 4, g] * ks[g]).max(0) for g in range(4)])
    assert np.allclose(sc, want_sc, rtol=1e-5, atol=1e-4)


def test_fused_head_norm_and_bf16_rounding():
    rng = np.random.default_rng(1)
    q = orc.to_bits(rng.standard_normal((16, 128)) * 2.0, orc.BF16)
    g1, g2 = orc.to_bits(rng.standard_normal(128) * 0.1, orc.BF16), orc.to_bits(rng.standard_normal(128) * 0.1, orc.BF16)
    k, ks, v, vs = util.int8_cache(rng, 2, 333, False)
    o, _ = orc.full_decode(q, orc.BF16, k, ks, v, vs, 333, gains=(g1, g2))
    qn = _f(orc.to_bits(_head_norm64(_f(q, orc.BF16), (g1, g2), orc.BF16), orc.BF16), orc.BF16)
    want = _relu2_64(qn, k, ks, v, vs, 8)
    ok, msg = util.close(orc.from_bits(o, orc.BF16), want, max_abs=4e-3, rel_rms=4e-3)   # bf16 output rounding
    assert ok, msg


def test_quantiser_properties():
    rng = np.random.default_rng(2)
    x = (rng.standard_normal((64, 128)) * rng.uniform(0.01, 30, (64, 1))).astype(np.float32)
    x[7] = 0.0
    xb = orc.to_bits(x, orc.BF16)
    codes, scales = orc.quantize_rows(xb, orc.BF16)
    xr = orc.from_bits(xb, orc.BF16)
    assert np.abs(codes).max() <= 127 and (np.abs(codes).max(1)[np.arange(64) != 7] == 127).all()
    assert (codes[7] == 0).all() and scales[7] == 0.0
    assert np.allclose(scales, np.abs(xr).max(1) / 127.0, rtol=1e-6)
    assert (np.abs(codes * scales[:, None] - xr) <= scales[:, None] * 0.5001 + 1e-12).all()   # round to nearest
    # keys are RMS-normed first (no gains): dequantised rows have unit RMS up to quantisation error
    codes_n, scales_n = orc.quantize_rows(xb, orc.BF16, norm=True)
    rms = np.sqrt(((codes_n * scales_n[:, None]) ** 2).mean(1))
    assert np.allclose(np.delete(rms, 7), 1.0, atol=2e-2)
    # fp16 scales are the fp32 ones rounded
    _, s16 = orc.quantize_rows(xb, orc.BF16, scale_f16=True)
    assert np.array_equal(s16, scales.astype(np.float16).astype(np.float32))


def _select_numpy(sc, S):
    out = []
    for row in sc:
        n = S - 128
        bits = np.array([orc.lib().orc_order_bits(float(x)) for x in row[:n]], dtype=np.uint64)
        order = np.lexsort((np.arange(n), -bits.astype(np.int64)))          # by key descending, then index ascending
        tau = bits[order[1023]]
        gt = np.nonzero(bits > tau)[0]
        eq = np.nonzero(bits == tau)[0][:1024 - len(gt)]
        out.append(np.concatenate([gt, eq, np.arange(n, S)]).astype(np.uint32))
    return np.stack(out)


def test_selection_ties_signed_zero_and_property():
    rng = np.random.default_rng(3)
    for S in (1153, 1500, 4000):
        sc = (np.round(rng.standard_normal((3, S)) * 2) / 2).astype(np.float32)   # heavy ties
        sc[0, ::5] = -0.0
        sc[0, 1::5] = 0.0
        sc[2] = -np.abs(sc[2]) - 1.0
        idx = orc.select_keys(sc, S)
        assert np.array_equal(idx, _select_numpy(sc, S))
        assert orc.verify_selection(sc, idx, S) == 0
        bad = idx.copy()
        bad[1, 3] = bad[1, 4]
        assert orc.verify_selection(sc, bad, S) == 1           # repeated rows
        bad = idx.copy()
        bad[0, 1024] += 1
        assert orc.verify_selection(sc, bad, S) in (1, 2)      # recent rows
    assert orc.lib().orc_order_bits(0.0) > orc.lib().orc_order_bits(-0.0)


def test_sparse_decode_vs_float64():
    rng = np.random.default_rng(4)
    S = 1300
    q = orc.to_bits(rng.standard_normal((16, 128)), orc.F16)
    kb = orc.to_bits(rng.standard_normal((4, S, 128)), orc.F16)
    vb = orc.to_bits(rng.standard_normal((4, S, 128)), orc.F16)
    sc = orc.score_keys(q, orc.F16, kb, S)
    idx = orc.select_keys(sc, S)
    o = orc.from_bits(orc.sparse_decode(q, orc.F16, kb, None, vb, None, S, idx=idx, kv_kind=1), orc.F16)
    qf, kf, vf = _f(q, orc.F16), _f(kb, orc.F16), _f(vb, orc.F16)
    for h in (0, 5, 15):
        rows = idx[h // 4].astype(np.int64)
        s = kf[h // 4][rows] @ qf[h] / np.sqrt(128.0)
        w = np.exp(s - s.max())
        want = w @ vf[h // 4][rows] / w.sum()
        ok, msg = util.close(o[h], want)
        assert ok, msg
    # scores = max over the group's heads of the raw dot
    want_sc = np.stack([(kf[g] @ qf[4 * g:4 * g + 4].T).max(1) for g in range(4)])
    assert np.allclose(sc[:, :S], want_sc, rtol=1e-5, atol=1e-4)


def test_sliding_norm_rope_ring_vs_float64():
    rng = np.random.default_rng(5)
    W, RING, dtype = 128, 256, orc.BF16
    qg, kg = orc.to_bits(rng.standard_normal(128) * 0.1, dtype), orc.to_bits(rng.standard_normal(128) * 0.1, dtype)
    T = 300                                       # wraps the ring
    k = orc.to_bits(rng.standard_normal((T, 4, 128)), dtype)
    v = orc.to_bits(rng.standard_normal((T, 4, 128)), dtype)
    rk, rv = np.zeros((4, RING, 128), np.uint16), np.zeros((4, RING, 128), np.uint16)
    orc.sliding_write(k, v, dtype, rk, rv, 0, kgain=kg)
    q = orc.to_bits(rng.standard_normal((1, 16, 128)), dtype)
    pos = T - 1
    o = orc.from_bits(orc.sliding_attend(q, dtype, rk, rv, pos, W, qgain=qg), dtype)[0]
    kn = np.stack([_rope64(_head_norm64(_f(k[t], dtype), (kg,), dtype), t) for t in range(T)])        # [T, 4, 128]
    kn = _f(orc.to_bits(kn, dtype), dtype)
    assert np.array_equal(orc.to_bits(kn[T - 1], dtype), rk[:, (T - 1) % RING])                        # slot = pos % RING
    qn = _f(orc.to_bits(_rope64(_head_norm64(_f(q[0], dtype), (qg,), dtype), pos), dtype), dtype)
    for h in (0, 7, 15):
        keys = np.arange(pos - W + 1, pos + 1)
        s = kn[keys, h // 4] @ qn[h] / np.sqrt(128.0)
        w = np.exp(s - s.max())
        want = w @ _f(v, dtype)[keys, h // 4] / w.sum()
        ok, msg = util.close(o[h], want, max_abs=4e-3, rel_rms=5e-3)   # bf16 rounding of q, k and o
        assert ok, msg


def test_prefill_rows_equal_decode_at_their_position():
    rng = np.random.default_rng(6)
    p0, Tq = 70, 9
    q = orc.to_bits(rng.standard_normal((Tq, 16, 128)), orc.BF16)
    k, ks, v, vs = util.int8_cache(rng, 4, p0 + Tq, True)
    o = orc.full_prefill(q, orc.BF16, k, ks, v, vs, p0)
    for r in (0, 4, 8):
        od, _ = orc.full_decode(q[r], orc.BF16, k, ks, v, vs, p0 + r + 1)
        assert np.array_equal(o[r], od)
    sub = orc.full_prefill(q, orc.BF16, k, ks, v, vs, p0, r0=1, rstep=3)
    assert np.array_equal(sub[1::3], o[1::3]) and (sub[0] == 0).all()


def test_golden_fixtures_are_reproduced(gold):
    g = gold
    c, s = orc.quantize_rows(g["quant_x"], orc.BF16, norm=True)
    assert np.array_equal(c, g["quant_codes_norm"]) and np.array_equal(s, g["quant_scales_norm"])
    c, s = orc.quantize_rows(g["quant_x"], orc.BF16, norm=False)
    assert np.array_equal(c, g["quant_codes_plain"]) and np.array_equal(s, g["quant_scales_plain"])
    S = g["full_k"].shape[1]
    o, sc = orc.full_decode(g["full_q"], orc.F16, g["full_k"], g["full_ks"], g["full_v"], g["full_vs"], S, want_scores=True)
    assert np.array_equal(o, g["full_o"]) and np.array_equal(sc.view(np.uint32), g["full_scores"].view(np.uint32))
    S = g["ref_k"].shape[1]
    o, sc = orc.full_decode(g["ref_q"], orc.BF16, g["ref_k"], g["ref_ks"], g["ref_v"], g["ref_vs"], S,
                            gains=(g["ref_g1"], g["ref_g2"]), want_scores=True)
    assert np.array_equal(o, g["ref_o"]) and np.array_equal(sc.view(np.uint32), g["ref_scores"].view(np.uint32))
    assert np.array_equal(orc.select_keys(g["sel_scores"], g["sel_scores"].shape[1]), g["sel_idx"])
    for name in ("sparse_short", "sparse_sel"):
        S = g[name + "_k"].shape[1]
        sc = orc.score_keys(g[name + "_q"], orc.F16, g[name + "_k"], S)
        assert np.array_equal(sc.view(np.uint32), g[name + "_scores"].view(np.uint32))
        idx = g[name + "_idx"] if name + "_idx" in g.files else None
        o = orc.sparse_decode(g[name + "_q"], orc.F16, g[name + "_k"], None, g[name + "_v"], None, S, idx=idx, kv_kind=1)
        assert np.array_equal(o, g[name + "_o"])
    rk, rv = np.zeros_like(g["slide_ring_k"]), np.zeros_like(g["slide_ring_v"])
    orc.sliding_write(g["slide_hist_k"], g["slide_hist_v"], orc.BF16, rk, rv, 0, kgain=g["slide_kg"])
    assert np.array_equal(rk, g["slide_ring_k"]) and np.array_equal(rv, g["slide_ring_v"])
    o = orc.sliding_attend(g["slide_q"], orc.BF16, rk, rv, g["slide_hist_k"].shape[0] - 1, 128, qgain=g["slide_qg"])
    assert np.array_equal(o, g["slide_o"])
    o = orc.full_prefill(g["pre_q"], orc.BF16, g["pre_k"], g["pre_ks"], g["pre_v"], g["pre_vs"], int(g["pre_p0"]))
    assert np.array_equal(o, g["pre_o"])


def test_w4_gemv_against_the_dequantised_matrix():
    """The 4-bit GEMV restatement (GemvRows: word c, part k, nibble n = column 32 c + 8 k + n; y = sum of scale * nibble dot
    + bias * sum of x per 64 columns) against x @ (scale * nibbles + bias) in float64."""
    rng = np.random.default_rng(12)
    rows, d_in, tokens = 24, 256, 5
    words = rng.integers(0, 2 ** 32, (rows, d_in // 32, 4), dtype=np.uint64).astype(np.uint32)
    sc = orc.to_bits(rng.uniform(0.002, 0.01, (rows, d_in // 64)), orc.BF16)
    bs = orc.to_bits(rng.standard_normal((rows, d_in // 64)) * 0.03, orc.BF16)
    xb = orc.to_bits(rng.standard_normal((tokens, d_in)), orc.BF16)
    for dtype in (orc.BF16, orc.F16):
        xd = orc.to_bits(orc.from_bits(xb, orc.BF16), dtype)
        y = orc.from_bits(orc.w4_gemv(words, sc, bs, xd, dtype), dtype).astype(np.float64)
        nib = np.zeros((rows, d_in))
        for c in range(d_in // 32):
            for k in range(4):
                for n in range(8):
                    nib[:, 32 * c + 8 * k + n] = (words[:, c, k] >> np.uint32(4 * n)) & np.uint32(15)
        w = np.repeat(orc.from_bits(sc, orc.BF16).astype(np.float64), 64, axis=1) * nib + \
            np.repeat(orc.from_bits(bs, orc.BF16).astype(np.float64), 64, axis=1)
        ref = orc.from_bits(xd, dtype).astype(np.float64) @ w.T
        step = 2.0 ** -8 if dtype == orc.BF16 else 2.0 ** -11            # half a step of the storage dtype
        assert np.all(np.abs(y - ref) <= step * np.abs(ref) + 1e-5)
