"""GPU test of the prefix store: a hit restores bytes identical to the sequence that was saved, and decoding from
the restored caches reproduces decoding from the original ones bit for bit (the check of the reference's
`embla-bench cache`, Sources/EmblaBench/Cache.swift:60-69)."""
import numpy as np
import pytest

from oracle import prefix_oracle as po

pytestmark = pytest.mark.gpu

HQ, HKV, N_FULL, N_SLIDE, RING, W = 16, 4, 2, 2, 1024, 128


def _setup(n_blocks=32):
    import torch
    from embla_metal_b200 import attn
    ctx = attn.Attention(HQ, HKV, attn.F16, max_batch=2, max_context=2048)
    pool = attn.KVPool(N_FULL, HKV, n_blocks, attn.KV_INT8, attn.SCALE_F16)
    pool.raw().view(-1).zero_()
    rings = [attn.Ring(2, HKV, RING, W, torch.float16) for _ in range(N_SLIDE)]
    return ctx, pool, rings


def _fill(ctx, pool, rings, seq, ids, n_pos, seed, pos0=0, total=700):
    """Appends positions pos0 .. n_pos - 1 of sequence `seq` to every layer; the k/v row of a position depends on `seed`
    and the position only (the rows of all `total` positions are drawn at once)."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(seed)
    table = torch.zeros(2, 16, dtype=torch.int32, device="cuda")
    table[seq, :len(ids)] = torch.tensor(ids, dtype=torch.int32, device="cuda")
    n_layers = N_FULL + N_SLIDE
    kv = torch.randn(n_layers, 2, total, HKV * 128, device="cuda", generator=g).half()[:, :, :n_pos]    # [layer][k|v][pos][...]
    p0 = torch.tensor([pos0, pos0], dtype=torch.int32, device="cuda")
    T = n_pos - pos0
    for l in range(N_FULL):
        k = torch.zeros(2, T, HKV * 128, dtype=torch.float16, device="cuda")
        v = torch.zeros_like(k)
        k[seq], v[seq] = kv[l, 0, pos0:], kv[l, 1, pos0:]
        # (the other sequence's row of the table points at block 0..: append only to `seq` by a batch-1 view)
        ctx.kv_append(pool, table[seq:seq + 1], l, p0[:1], k[seq:seq + 1], v[seq:seq + 1])
    for r in range(N_SLIDE):
        k = torch.zeros(2, T, HKV * 128, dtype=torch.float16, device="cuda")
        v = torch.zeros_like(k)
        k[seq], v[seq] = kv[N_FULL + r, 0, pos0:], kv[N_FULL + r, 1, pos0:]
        ring = rings[r]
        one = type("R", (), {})()
        from embla_metal_b200 import attn
        one.desc = attn.RingDesc(ring.k[seq].data_ptr(), ring.v[seq].data_ptr(), ring.k.stride(0), RING, W)
        ctx.sliding_write(one, p0[:1], k[seq:seq + 1], v[seq:seq + 1])
    torch.cuda.synchronize()
    return table


def _decode(ctx, pool, rings, table, seq, S, seed):
    import torch
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(1, HQ * 128, device="cuda", generator=g).half()
    lens = torch.tensor([S], dtype=torch.int32, device="cuda")
    outs = []
    for l in range(N_FULL):
        o = torch.zeros_like(q)
        ctx.full_decode(pool, table[seq:seq + 1], lens, l, q, o, max_seq_len=S)
        outs.append(o)
    from embla_metal_b200 import attn
    for ring in rings:
        one = type("R", (), {})()
        one.desc = attn.RingDesc(ring.k[seq].data_ptr(), ring.v[seq].data_ptr(), ring.k.stride(0), RING, W)
        o = torch.zeros_like(q)
        ctx.sliding_decode(one, lens, q, o)
        outs.append(o)
    ctx.check()
    return torch.cat(outs).view(torch.int16).cpu().numpy()


def test_hit_restores_identical_bytes_and_decodes_identically():
    import torch
    from embla_metal_b200 import prefix
    ctx, pool, rings = _setup()
    rng = np.random.default_rng(3)
    tokens = [int(x) for x in rng.integers(0, 50000, 700)]
    ids_a, ids_b = [5, 2, 9, 0, 7, 3], [11, 12, 13, 14, 15, 16]
    table_a = _fill(ctx, pool, rings, 0, ids_a, 700, seed=1)
    store = prefix.PrefixStore(1 << 30, pool=pool, rings=rings, n_kv_heads=HKV)
    orc = po.PrefixOracle(1 << 30, store.full_block_bytes, store.window_bytes, ring=RING)
    store.save(0, ids_a, tokens, 700, [650, 700], 0)
    new_blocks, new_windows = orc.save(tokens, 700, [650, 700], 0)
    assert new_blocks == [0, 1, 2, 3, 4] and new_windows == [3, 4]
    s = store.stats()
    assert s["blocks"] == 5 and s["checkpoints"] == 2 and s["bytes"] == orc.bytes

    # another conversation that starts with the first 660 tokens
    prompt = tokens[:660] + [int(x) for x in rng.integers(0, 50000, 40)]
    start, valid = store.restore(1, ids_b, prompt, live=0, reuse=0)
    assert (start, valid) == (640, 512) and orc.restore(prompt, 0, 0)[0] == 640
    torch.cuda.synchronize()
    raw = pool.raw()
    for j in range(5):
        assert torch.equal(raw[ids_b[j]], raw[ids_a[j]]), f"block {j}"
    assert not raw[ids_b[5]].any(), "blocks past the resume point stay untouched"
    for ring in rings:
        for t in (ring.k, ring.v):
            assert torch.equal(t[1, :, 512:640], t[0, :, 512:640])
            assert not t[1, :, :512].any() and not t[1, :, 640:].any(), "only the checkpoint's 128 slots are written"

    # the restored sequence computes positions 640..659 as the original did, then both decode at 660 keys
    table_b = _fill(ctx, pool, rings, 1, ids_b, 660, seed=1, pos0=640)
    a = _decode(ctx, pool, rings, table_a, 0, 660, seed=9)
    b = _decode(ctx, pool, rings, table_b, 1, 660, seed=9)
    assert np.array_equal(a, b), "decoding from the restored caches differs from decoding from the original ones"
    store.close()
    pool.close()
    ctx.close()


def test_eviction_reuses_slots_and_keeps_data_right():
    import torch
    from embla_metal_b200 import prefix
    ctx, pool, rings = _setup()
    rng = np.random.default_rng(4)
    tok_a = [int(x) for x in rng.integers(0, 50000, 300)]
    tok_c = [int(x) for x in rng.integers(0, 50000, 300)]
    ids_a, ids_c, ids_b = [1, 2, 3], [4, 5, 6], [7, 8, 9]
    _fill(ctx, pool, rings, 0, ids_a, 300, seed=11)
    probe = prefix.PrefixStore(1, pool=pool, rings=rings, n_kv_heads=HKV)
    limit = 2 * probe.full_block_bytes + probe.window_bytes            # room for one 2-block sequence with its checkpoint
    probe.close()
    store = prefix.PrefixStore(limit, pool=pool, rings=rings, n_kv_heads=HKV)
    orc = po.PrefixOracle(limit, store.full_block_bytes, store.window_bytes, ring=RING)
    store.save(0, ids_a, tok_a, 300, [300], 0)
    orc.save(tok_a, 300, [300], 0)
    assert store.stats()["checkpoints"] == 1 and store.stats()["bytes"] == limit
    # a second sequence pushes the first one out; its slots are handed to the new blocks
    for ring in rings:
        ring.k.zero_()
        ring.v.zero_()
    _fill(ctx, pool, rings, 0, ids_c, 300, seed=12)
    store.save(0, ids_c, tok_c, 300, [300], 0)
    orc.save(tok_c, 300, [300], 0)
    s = store.stats()
    assert s["evicted"] == orc.evicted == 2 and s["bytes"] == orc.bytes == limit
    assert store.restore(1, ids_b, tok_a + [1], 0, 0) == (None, None)
    start, valid = store.restore(1, ids_b, tok_c + [1], 0, 0)
    assert (start, valid) == (256, 128)
    torch.cuda.synchronize()
    raw = pool.raw()
    assert torch.equal(raw[ids_b[0]], raw[ids_c[0]]) and torch.equal(raw[ids_b[1]], raw[ids_c[1]])
    for ring in rings:
        assert torch.equal(ring.k[1, :, 128:256], ring.k[0, :, 128:256]) and torch.equal(ring.v[1, :, 128:256], ring.v[0, :, 128:256])
    store.close()
    pool.close()
    ctx.close()
