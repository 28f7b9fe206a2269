"""ctypes binding of the CPU oracle (oracle/embla_oracle.cpp). TEST INFRASTRUCTURE.

Only the tests, the smoke check and the bench's CPU-baseline legs import this module; the product
(the CUDA library and its host wrapper) never does. 16-bit activations travel as raw uint16 numpy
arrays together with a dtype flag (BF16 = 0, F16 = 1).
"""
import ctypes as C
import os
import subprocess

import numpy as np

BF16, F16 = 0, 1
TOPK, RECENT = 1024, 128
HD = 128
_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build():
    """Compile the oracle with its Makefile (g++ only)."""
    subprocess.run(["make", "-s", "-C", _HERE], check=True)


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "libembla_oracle.so")
        if not os.path.exists(path):
            build()
        _LIB = C.CDLL(path)
        _LIB.orc_round_act.restype = C.c_float
        _LIB.orc_round_act.argtypes = [C.c_float, C.c_int]
        _LIB.orc_order_bits.restype = C.c_uint32
        _LIB.orc_order_bits.argtypes = [C.c_float]
    return _LIB


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dt):
    return None if a is None else np.ascontiguousarray(a, dtype=dt)


# ---- 16-bit storage helpers -----------------------------------------------------------------
def to_bits(x, dtype):
    """float array -> uint16 storage of `dtype` (round to nearest even)."""
    x = np.asarray(x, dtype=np.float32)
    if dtype == F16:
        return x.astype(np.float16).view(np.uint16)
    u = x.view(np.uint32).astype(np.uint64)
    return (((u + (((u >> 16) & 1) + 0x7FFF)) >> 16) & 0xFFFF).astype(np.uint16)


def from_bits(b, dtype):
    b = np.asarray(b, dtype=np.uint16)
    if dtype == F16:
        return b.view(np.float16).astype(np.float32)
    return (b.astype(np.uint32) << 16).view(np.float32)


# ---- oracle entry points ----------------------------------------------------------------------
def quantize_rows(x_bits, dtype, norm=False, scale_f16=False):
    x = _c(x_bits, np.uint16).reshape(-1, HD)
    n = x.shape[0]
    codes = np.empty((n, HD), np.int8)
    scales = np.empty(n, np.float32)
    lib().orc_quantize_rows(_p(x), n, dtype, int(norm), int(scale_f16), _p(codes), _p(scales))
    return codes, scales


def _kv(kv_kind, k, ks, v, vs):
    if kv_kind == 0:
        return _c(k, np.int8), _c(ks, np.float32), _c(v, np.int8), _c(vs, np.float32)
    return _c(k, np.uint16), None, _c(v, np.uint16), None


def full_decode(q_bits, dtype, k, ks, v, vs, S, kv_kind=0, gains=None, want_scores=False):
    """q [Hq,128]; k, v [Hkv, ldS, 128]; ks, vs [Hkv, ldS]. Returns (o_bits [Hq,128], scores or None)."""
    q = _c(q_bits, np.uint16)
    Hq, Hkv, ldS = q.shape[0], k.shape[0], k.shape[1]
    k, ks, v, vs = _kv(kv_kind, k, ks, v, vs)
    g1 = g2 = None
    ng = 0
    if gains is not None:
        g1, g2 = _c(gains[0], np.uint16), _c(gains[1], np.uint16)
        ng = 2
    o = np.empty((Hq, HD), np.uint16)
    scores = np.zeros((Hkv, ldS), np.float32) if want_scores else None
    lib().orc_full_decode(_p(q), dtype, int(gains is None), _p(g1), _p(g2), ng, kv_kind, _p(k), _p(ks), _p(v), _p(vs),
                          Hq, Hkv, S, ldS, _p(o), _p(scores))
    return o, scores


def score_keys(q_bits, dtype, k, S, kv_kind=1, ks=None, nthreads=1):
    q = _c(q_bits, np.uint16)
    Hq, Hkv, ldS = q.shape[0], k.shape[0], k.shape[1]
    k = _c(k, np.int8 if kv_kind == 0 else np.uint16)
    ks = _c(ks, np.float32)
    scores = np.zeros((Hkv, ldS), np.float32)
    lib().orc_score_keys(_p(q), dtype, kv_kind, _p(k), _p(ks), Hq, Hkv, S, ldS, _p(scores), nthreads)
    return scores


def select_keys(scores, S):
    scores = _c(scores, np.float32)
    Hkv, ldS = scores.shape
    idx = np.empty((Hkv, TOPK + RECENT), np.uint32)
    lib().orc_select_keys(_p(scores), Hkv, S, ldS, _p(idx))
    return idx


def verify_selection(scores, idx, S):
    scores = _c(scores, np.float32)
    idx = _c(idx, np.uint32)
    Hkv, ldS = scores.shape
    return lib().orc_verify_selection(_p(scores), _p(idx), Hkv, S, ldS)


def sparse_decode(q_bits, dtype, k, ks, v, vs, S, idx=None, kv_kind=0, gains=None):
    q = _c(q_bits, np.uint16)
    Hq, Hkv, ldS = q.shape[0], k.shape[0], k.shape[1]
    k, ks, v, vs = _kv(kv_kind, k, ks, v, vs)
    g1 = g2 = None
    ng = 0
    if gains is not None:
        g1, g2 = _c(gains[0], np.uint16), _c(gains[1], np.uint16)
        ng = 2
    idx = _c(idx, np.uint32)
    nsel = 0 if idx is None else idx.shape[1]
    o = np.empty((Hq, HD), np.uint16)
    lib().orc_sparse_decode(_p(q), dtype, int(gains is None), _p(g1), _p(g2), ng, kv_kind, _p(k), _p(ks), _p(v), _p(vs),
                            Hq, Hkv, S, ldS, _p(idx), nsel, _p(o))
    return o


def sliding_write(k_bits, v_bits, dtype, ring_k, ring_v, p0, kgain=None):
    """k, v [T, Hkv, 128]; ring_k, ring_v [Hkv, RING, 128] uint16, updated in place."""
    k, v = _c(k_bits, np.uint16), _c(v_bits, np.uint16)
    T, Hkv = k.shape[0], k.shape[1]
    assert ring_k.flags.c_contiguous and ring_v.flags.c_contiguous
    kg = _c(kgain, np.uint16)
    lib().orc_sliding_write(_p(k), _p(v), Hkv * HD, T, dtype, int(kgain is None), _p(kg), _p(ring_k), _p(ring_v),
                            p0, ring_k.shape[1], Hkv)


def sliding_attend(q_bits, dtype, ring_k, ring_v, p0, W, qgain=None, nthreads=1):
    """q [T, Hq, 128] -> o [T, Hq, 128]."""
    q = _c(q_bits, np.uint16)
    T, Hq = q.shape[0], q.shape[1]
    Hkv, RING = ring_k.shape[0], ring_k.shape[1]
    qg = _c(qgain, np.uint16)
    o = np.empty((T, Hq, HD), np.uint16)
    lib().orc_sliding_attend(_p(q), Hq * HD, T, dtype, int(qgain is None), _p(qg), _p(ring_k), _p(ring_v), p0, W, RING,
                             Hq, Hkv, _p(o), nthreads)
    return o


def full_prefill(q_bits, dtype, k, ks, v, vs, p0, kv_kind=0, gains=None, r0=0, rstep=1, nthreads=1, want_f32=False, qk8=False):
    """q [Tq, Hq, 128]; caches [Hkv, ldS, 128] holding p0 + Tq keys. Returns o [Tq, Hq, 128]
    (rows outside r0::rstep are zero); with want_f32 also the unrounded fp32 results. qk8: the reference's int8 Q Kᵀ
    build (query rows quantised like cache rows, integer dots; int8 cache only)."""
    q = _c(q_bits, np.uint16)
    Tq, Hq = q.shape[0], q.shape[1]
    Hkv, ldS = k.shape[0], k.shape[1]
    k, ks, v, vs = _kv(kv_kind, k, ks, v, vs)
    g1 = g2 = None
    if gains is not None:
        g1, g2 = _c(gains[0], np.uint16), _c(gains[1], np.uint16)
    o = np.zeros((Tq, Hq, HD), np.uint16)
    o32 = np.zeros((Tq, Hq, HD), np.float32) if want_f32 else None
    if qk8:
        assert kv_kind == 0
        lib().orc_full_prefill_qk8(_p(q), Hq * HD, Tq, dtype, int(gains is None), _p(g1), _p(g2), _p(k), _p(ks), _p(v),
                                   _p(vs), Hq, Hkv, p0, ldS, _p(o), r0, rstep, nthreads, _p(o32))
    else:
        lib().orc_full_prefill(_p(q), Hq * HD, Tq, dtype, int(gains is None), _p(g1), _p(g2), kv_kind, _p(k), _p(ks), _p(v),
                               _p(vs), Hq, Hkv, p0, ldS, _p(o), r0, rstep, nthreads, _p(o32))
    return (o, o32) if want_f32 else o


def full_decode_batch(q_bits, dtype, k, ks, v, vs, S, nthreads):
    """q [B, Hq, 128]; k, v [B, Hkv, ldS, 128] int8; ks, vs [B, Hkv, ldS]. Returns o [B, Hq, 128]."""
    q = _c(q_bits, np.uint16)
    B, Hq = q.shape[0], q.shape[1]
    Hkv, ldS = k.shape[1], k.shape[2]
    k, ks, v, vs = _kv(0, k, ks, v, vs)
    o = np.empty((B, Hq, HD), np.uint16)
    lib().orc_full_decode_batch(B, nthreads, _p(q), dtype, _p(k), _p(ks), _p(v), _p(vs), Hq, Hkv, S, ldS, _p(o))
    return o


def w4_gemv(words, scales, biases, x_bits, dtype, nthreads=1):
    """words [rows, d_in / 32, 4] uint32, scales / biases [rows, d_in / 64] bfloat16 bits, x [tokens, d_in] storage bits.
    Returns y [tokens, rows] storage bits."""
    words = _c(words, np.uint32)
    scales, biases, x = _c(scales, np.uint16), _c(biases, np.uint16), _c(x_bits, np.uint16)
    rows, d_in, tokens = words.shape[0], words.shape[1] * 32, x.shape[0]
    y = np.empty((tokens, rows), np.uint16)
    lib().orc_w4_gemv(_p(words), _p(scales), _p(biases), rows, d_in, _p(x), x.shape[1], tokens, dtype, _p(y), rows, nthreads)
    return y
