"""GPU parity of key scoring, key selection, sparse-layer decode and sliding-layer decode against the
CPU oracle, through the C ABI. Index sets are compared bit for bit, in the reference's output order."""
import numpy as np
import pytest

from oracle import oracle as orc
from tests import util

pytestmark = pytest.mark.gpu


def _pool16(attn, rng, k_bits, v_bits, Hkv, extra_layers=1):
    """A 16-bit pool holding one sequence's K, V [Hkv, S, 128] (uint16) at shuffled blocks of layer 1."""
    import torch
    S = k_bits.shape[1]
    npg = (S + 127) // 128
    pool = attn.KVPool(1 + extra_layers, Hkv, npg + 2, attn.KV_16BIT)
    ids = rng.permutation(npg + 2)[:npg].astype(np.int32)
    raw = pool.raw()
    pad = np.zeros((Hkv, npg * 128, 128), np.uint16)
    padv = np.zeros_like(pad)
    pad[:, :S] = k_bits
    padv[:, :S] = v_bits
    pages = np.concatenate([pad.reshape(Hkv, npg, 128 * 128), padv.reshape(Hkv, npg, 128 * 128)], axis=2)
    t = torch.from_numpy(pages.view(np.uint8).reshape(Hkv, npg, 65536)).cuda()
    raw[torch.as_tensor(ids, device="cuda", dtype=torch.long), 1] = t.permute(1, 0, 2)
    return pool, ids


def _sparse_case(S, Hq, Hkv, dtype, seed, gains=False, boost=True):
    import torch
    from embla_metal_b200 import attn
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((Hq, 128)).astype(np.float32)
    k = rng.standard_normal((Hkv, S, 128)).astype(np.float32)
    if boost:   # 1 % of the keys scaled x4 so the top-k is not trivial
        k[:, rng.random(S) < 0.01] *= 4.0
    v = rng.standard_normal((Hkv, S, 128)).astype(np.float32)
    qb, kb, vb = orc.to_bits(q, dtype), orc.to_bits(k, dtype), orc.to_bits(v, dtype)
    g = None
    if gains:
        g = (orc.to_bits(rng.standard_normal(128) * 0.1, dtype), orc.to_bits(rng.standard_normal(128) * 0.1, dtype))
    ctx = attn.Attention(Hq, Hkv, dtype, max_batch=1, max_context=(S + 127) // 128 * 128)
    pool, ids = _pool16(attn, rng, kb, vb, Hkv)
    tbl = torch.from_numpy(ids[None]).cuda()
    lens = torch.tensor([S], dtype=torch.int32, device="cuda")
    qt = util.act_tensor(qb.reshape(1, Hq * 128), dtype)
    ldS = (S + 127) // 128 * 128
    scores = torch.full((1, Hkv, ldS), -3.0, device="cuda")
    ctx.score_keys(pool, tbl, lens, 1, qt, scores, max_seq_len=S)
    want_sc = orc.score_keys(qb, dtype, kb, S)
    got_sc = scores[0, :, :S].cpu().numpy()
    assert np.array_equal(got_sc.view(np.uint32), want_sc[:, :S].view(np.uint32)), "scores are not bit-exact"
    idx_t = None
    want_idx = None
    if S > 1152:
        idx_t = torch.zeros((1, Hkv, 1152), dtype=torch.int32, device="cuda")
        ctx.select_keys(scores, lens, idx_t, max_seq_len=S)
        want_idx = orc.select_keys(want_sc, S)
        got_idx = idx_t[0].cpu().numpy().view(np.uint32)
        assert np.array_equal(got_idx, want_idx), "selected rows differ"
        assert orc.verify_selection(want_sc, got_idx, S) == 0
    ot = torch.zeros_like(qt)
    gt = None if g is None else (util.act_tensor(g[0], dtype), util.act_tensor(g[1], dtype))
    ctx.sparse_decode(pool, tbl, lens, 1, qt, ot, idx=idx_t, gains=gt, max_seq_len=S)
    ctx.check()
    want_o = orc.from_bits(orc.sparse_decode(qb, dtype, kb, None, vb, None, S, idx=want_idx, kv_kind=1, gains=g), dtype)
    got_o = orc.from_bits(util.act_bits(ot), dtype).reshape(Hq, 128)
    ok, msg = util.close(got_o, want_o)
    assert ok, f"sparse decode S={S}: {msg}"
    ot2 = torch.zeros_like(qt)
    ctx.sparse_decode(pool, tbl, lens, 1, qt, ot2, idx=idx_t, gains=gt, max_seq_len=S)
    torch.cuda.synchronize()
    assert torch.equal(ot.view(torch.int16), ot2.view(torch.int16))
    pool.close()
    ctx.close()


def test_config2_sparse_32k():
    # benchmark configuration 2: 32768 context, fp16, 1 % of keys x4, seed 2
    _sparse_case(32768, 16, 4, orc.F16, seed=2)


@pytest.mark.parametrize("S", [1, 5, 128, 129, 511, 513, 1151, 1152, 1153, 1300, 4096])
def test_sparse_lengths(S):
    _sparse_case(S, 16, 4, orc.F16, seed=100 + S)


def test_sparse_bf16_two_kv_heads_gains():
    _sparse_case(2000, 16, 2, orc.BF16, seed=9, gains=True)
    _sparse_case(700, 16, 2, orc.BF16, seed=10, gains=True)


def test_select_ties_and_signed_zero():
    """Ties at the 1024-th score (lowest indices win), negative scores, +0 above -0, batch of 3."""
    import torch
    from embla_metal_b200 import attn
    rng = np.random.default_rng(33)
    Hkv, S_list = 4, [1153, 3000, 900]
    ld = 3072
    ctx = attn.Attention(16, Hkv, orc.F16, max_batch=3, max_context=ld)
    scores = np.zeros((3, Hkv, ld), np.float32)
    scores[0] = rng.integers(-3, 4, (Hkv, ld)).astype(np.float32)            # massive ties
    scores[1] = np.round(rng.standard_normal((Hkv, ld)) * 4) / 4
    scores[1, 0, ::2] = -0.0
    scores[1, 1] = -np.abs(scores[1, 1])                                      # all negative
    scores[1, 2, :] = 1.0                                                     # all equal
    scores[2] = rng.standard_normal((Hkv, ld))
    st = torch.from_numpy(scores).cuda()
    lens = torch.tensor(S_list, dtype=torch.int32, device="cuda")
    idx = torch.full((3, Hkv, 1152), -1, dtype=torch.int32, device="cuda")
    ctx.select_keys(st, lens, idx, max_seq_len=max(S_list))
    torch.cuda.synchronize()
    got = idx.cpu().numpy()
    for b, S in enumerate(S_list):
        if S <= 1152:
            assert (got[b] == -1).all(), "short sequences must be left untouched"
            continue
        want = orc.select_keys(scores[b], S)
        assert np.array_equal(got[b].view(np.uint32), want), f"sequence {b}"
        assert orc.verify_selection(scores[b], got[b].view(np.uint32), S) == 0
    ctx.close()


def _sliding_case(pos_list, W, RING, dtype, seed, gains, poison=False):
    import torch
    from embla_metal_b200 import attn
    rng = np.random.default_rng(seed)
    Hq, Hkv, B = 16, 4, len(pos_list)
    ctx = attn.Attention(Hq, Hkv, dtype, max_batch=B, max_context=RING)
    tdt = torch.bfloat16 if dtype == orc.BF16 else torch.float16
    ring = attn.Ring(B, Hkv, RING, W, tdt)
    qg = kg = None
    if gains:
        qg = orc.to_bits(rng.standard_normal(128) * 0.1, dtype)
        kg = orc.to_bits(rng.standard_normal(128) * 0.1, dtype)
    want = []
    # slots no token has been written to: zeros, or (poison) NaN bit patterns as uninitialised memory may hold
    rk_all = np.full((B, Hkv, RING, 128), 0x7FFF if poison else 0, np.uint16)
    rv_all = np.full((B, Hkv, RING, 128), 0x7FFF if poison else 0, np.uint16)
    q = orc.to_bits(rng.standard_normal((B, Hq, 128)), dtype)
    knew = orc.to_bits(rng.standard_normal((B, 1, Hkv, 128)), dtype)
    vnew = orc.to_bits(rng.standard_normal((B, 1, Hkv, 128)), dtype)
    for b, pos in enumerate(pos_list):
        # history: the last min(pos, RING) positions written through the oracle's ring write
        n_hist = min(pos, RING - 1)
        hk = orc.to_bits(rng.standard_normal((n_hist, Hkv, 128)), dtype)
        hv = orc.to_bits(rng.standard_normal((n_hist, Hkv, 128)), dtype)
        if n_hist:
            orc.sliding_write(hk, hv, dtype, rk_all[b], rv_all[b], pos - n_hist, kgain=kg)
    ring.k.copy_(util.act_tensor(rk_all, dtype))
    ring.v.copy_(util.act_tensor(rv_all, dtype))
    for b, pos in enumerate(pos_list):
        orc.sliding_write(knew[b], vnew[b], dtype, rk_all[b], rv_all[b], pos, kgain=kg)
        want.append(orc.from_bits(orc.sliding_attend(q[b][None], dtype, rk_all[b], rv_all[b], pos, W, qgain=qg), dtype)[0])
    pos_t = torch.tensor(pos_list, dtype=torch.int32, device="cuda")
    ctx.sliding_write(ring, pos_t, util.act_tensor(knew.reshape(B, 1, Hkv * 128), dtype),
                      util.act_tensor(vnew.reshape(B, 1, Hkv * 128), dtype),
                      kgain=None if kg is None else util.act_tensor(kg, dtype))
    torch.cuda.synchronize()
    # the ring write is elementwise arithmetic in the oracle's order: compare the stored rows closely
    written = rk_all != 0x7FFF if poison else np.ones(rk_all.shape, bool)
    gk = np.where(written, orc.from_bits(util.act_bits(ring.k), dtype), 0.0)
    wk = np.where(written, orc.from_bits(rk_all, dtype), 0.0)
    step = 2.0 ** -7 if dtype == orc.BF16 else 2.0 ** -10     # sin/cos may differ by an ulp: one storage step
    assert np.abs(gk - wk).max() <= step * max(1.0, np.abs(wk).max())
    assert np.array_equal(util.act_bits(ring.v), rv_all)
    qt = util.act_tensor(q.reshape(B, Hq * 128), dtype)
    ot = torch.zeros_like(qt)
    lens = pos_t + 1
    ctx.sliding_decode(ring, lens, qt, ot, qgain=None if qg is None else util.act_tensor(qg, dtype))
    ctx.check()
    got = orc.from_bits(util.act_bits(ot), dtype).reshape(B, Hq, 128)
    for b in range(B):
        ok, msg = util.close(got[b], want[b])
        assert ok, f"sliding decode pos={pos_list[b]}: {msg}"
    ctx.close()


def test_config1_sliding_decode():
    # benchmark configuration 1 (a): window 1024, ring 4096, fp16, decode at 4096 context (pos 4095), seed 1
    _sliding_case([4095], 1024, 4096, orc.F16, seed=1, gains=False)


def test_sliding_ring_boundary_and_short():
    _sliding_case([0, 1, 127, 128, 1023, 1024, 4096, 4097, 9000], 1024, 4096, orc.F16, seed=4, gains=False)


def test_sliding_reference_shape_norm_rope():
    # the reference's own window (128) with fused head norm + RoPE, bf16
    _sliding_case([0, 5, 200, 4095, 4096, 30000], 128, 4096, orc.BF16, seed=6, gains=True)


def test_sliding_unwritten_slots_hold_nans():
    # short sequences: most of the ring (and of the tiles the kernel fetches) was never written
    _sliding_case([0, 5, 70, 1000, 1023, 1024], 1024, 4096, orc.F16, seed=8, gains=False, poison=True)
    _sliding_case([3, 64, 127, 128, 129], 128, 4096, orc.BF16, seed=9, gains=True, poison=True)


def test_sliding_ring_not_a_multiple_of_64():
    # such rings are read row by row (gathered), not as 64-slot tiles
    _sliding_case([0, 299, 300, 999, 1000, 2500], 300, 1000, orc.F16, seed=10, gains=False, poison=True)


def test_select_large_batch_single_cta_path():
    """With many (sequence, kv head) pairs each pair is ranked by one CTA (small batches use a cluster of CTAs per pair)."""
    import torch
    from embla_metal_b200 import attn
    rng = np.random.default_rng(77)
    B, Hkv, ld = 40, 4, 2304
    S_list = [int(x) for x in rng.integers(1100, ld + 1, B)]
    ctx = attn.Attention(16, Hkv, orc.F16, max_batch=B, max_context=ld)
    scores = (np.round(rng.standard_normal((B, Hkv, ld)) * 8) / 8).astype(np.float32)
    st = torch.from_numpy(scores).cuda()
    lens = torch.tensor(S_list, dtype=torch.int32, device="cuda")
    idx = torch.full((B, Hkv, 1152), -1, dtype=torch.int32, device="cuda")
    ctx.select_keys(st, lens, idx, max_seq_len=ld)
    torch.cuda.synchronize()
    got = idx.cpu().numpy()
    for b, S in enumerate(S_list):
        if S <= 1152:
            assert (got[b] == -1).all()
        else:
            assert np.array_equal(got[b].view(np.uint32), orc.select_keys(scores[b], S)), f"sequence {b}"
    ctx.close()


@pytest.mark.parametrize("B", [2, 40])
def test_select_unaligned_rows_and_special_values(B):
    """Score rows that do not start on 16 bytes take the lanes' own loads instead of bulk copies; infinities and
    tiny/huge magnitudes rank by their order-preserving bit patterns as in the reference."""
    import torch
    from embla_metal_b200 import attn
    rng = np.random.default_rng(5 + B)
    Hkv, ld = 4, 4099                       # odd row stride: rows start at 4-byte offsets
    S_list = [int(x) for x in rng.integers(1153, ld + 1, B)]
    S_list[0] = ld
    ctx = attn.Attention(16, Hkv, orc.F16, max_batch=B, max_context=ld)
    scores = rng.standard_normal((B, Hkv, ld)).astype(np.float32) * np.float32(11.0)
    scores[0, 0, 5::97] = np.inf
    scores[0, 1, 3::89] = -np.inf
    scores[0, 2, ::3] *= np.float32(1e-30)
    scores[0, 3, ::5] *= np.float32(1e30)
    flat = torch.zeros(B * Hkv * ld + 1, dtype=torch.float32, device="cuda")
    st = flat[1:].view(B, Hkv, ld)          # 4 bytes past an aligned base
    st.copy_(torch.from_numpy(scores))
    assert st.data_ptr() % 16 == 4
    lens = torch.tensor(S_list, dtype=torch.int32, device="cuda")
    idx = torch.full((B, Hkv, 1152), -1, dtype=torch.int32, device="cuda")
    ctx.select_keys(st, lens, idx, max_seq_len=ld)
    ctx.check()
    got = idx.cpu().numpy()
    for b, S in enumerate(S_list):
        assert np.array_equal(got[b].view(np.uint32), orc.select_keys(scores[b], S)), f"sequence {b}"
    ctx.close()


@pytest.mark.parametrize("dtype,Hkv,norm_k", [(orc.F16, 4, False), (orc.BF16, 2, True)])
def test_fused_append_in_scoring_equals_append_then_score(dtype, Hkv, norm_k):
    """embla_score_keys_step writes the same 16-bit rows and the same scores as embla_kv_append + embla_score_keys."""
    import torch
    from embla_metal_b200 import attn
    rng = np.random.default_rng(41)
    S_list = [1, 128, 129, 1153, 2000, 4097]
    B, Hq = len(S_list), 16
    npg = (max(S_list) + 127) // 128
    ctx = attn.Attention(Hq, Hkv, dtype, max_batch=B, max_context=npg * 128)
    tdt = torch.bfloat16 if dtype == orc.BF16 else torch.float16
    pools = [attn.KVPool(1, Hkv, B * npg, attn.KV_16BIT) for _ in range(2)]
    table = torch.from_numpy(rng.permutation(B * npg).reshape(B, npg).astype(np.int32)).cuda()
    pools[0].raw().view(tdt).copy_(torch.randn(pools[0].raw().view(tdt).shape, device="cuda").to(tdt))
    pools[1].raw().copy_(pools[0].raw())
    lens = torch.tensor(S_list, dtype=torch.int32, device="cuda")
    q = util.act_tensor(orc.to_bits(rng.standard_normal((B, Hq * 128)), dtype), dtype)
    k = util.act_tensor(orc.to_bits(rng.standard_normal((B, Hkv * 128)) * 2, dtype), dtype)
    v = util.act_tensor(orc.to_bits(rng.standard_normal((B, Hkv * 128)), dtype), dtype)
    sc0 = torch.zeros(B, Hkv, npg * 128, device="cuda")
    sc1 = torch.zeros_like(sc0)
    ctx.kv_append(pools[0], table, 0, lens - 1, k.view(B, 1, -1), v.view(B, 1, -1), norm_k=norm_k)
    ctx.score_keys(pools[0], table, lens, 0, q, sc0, max_seq_len=max(S_list))
    ctx.score_keys_step(pools[1], table, lens, 0, q, k, v, sc1, max_seq_len=max(S_list), norm_k=norm_k)
    ctx.check()
    assert torch.equal(pools[0].raw(), pools[1].raw()), "the fused append wrote other bytes"
    for b, S in enumerate(S_list):
        assert torch.equal(sc0[b, :, :S], sc1[b, :, :S]), f"scores of sequence {b} differ"
    for pool in pools:
        pool.close()
    ctx.close()
