"""The native prefix store's index against the CPU restatement of the reference's PrefixCache, without a GPU
(dry run: no device memory, no copies)."""
import numpy as np

from oracle import prefix_oracle as po

FULL, WIN = 1000, 4000     # byte sizes of a stored block and of a checkpoint in these tests


def _store(limit, ring=4096):
    from embla_metal_b200 import prefix
    return prefix.PrefixStore(limit, pool=None, rings=(), ring_slots=ring, dry_run=True, full_block_bytes=FULL, window_bytes=WIN)


def test_hash_is_chained_fnv1a():
    from embla_metal_b200 import prefix
    rng = np.random.default_rng(0)
    assert prefix.prefix_hash(0, []) == 0xCBF29CE484222325
    # one token 0x01020304: bytes 04 03 02 01, low byte first
    h = 0xCBF29CE484222325
    for byte in (4, 3, 2, 1):
        h = ((h ^ byte) * 0x100000001B3) & po.MASK
    assert prefix.prefix_hash(0, [0x01020304]) == h
    for _ in range(20):
        t = rng.integers(0, 200000, 128)
        parent = int(rng.integers(0, 2 ** 63))
        assert prefix.prefix_hash(parent, t) == po.fnv_hash(parent, [int(x) for x in t])


def _same_state(store, orc, probes):
    s = store.stats()
    assert s["bytes"] == orc.bytes and s["blocks"] == len(orc.blocks) and s["evicted"] == orc.evicted
    assert s["checkpoints"] == sum(b.window for b in orc.blocks.values())
    for t in probes:
        got = store.chain(t)
        want = [(b.hash, b.window) for b in orc.chain(t, len(t))]
        assert got == want


def test_save_restore_evict_follow_the_reference_rules():
    rng = np.random.default_rng(1)
    limit = 30 * FULL + 3 * WIN
    store, orc = _store(limit), po.PrefixOracle(limit, FULL, WIN)
    system = [int(x) for x in rng.integers(0, 50000, 700)]           # a shared instruction prefix
    convs = []
    for step in range(60):
        if convs and rng.random() < 0.5:
            base = convs[int(rng.integers(0, len(convs)))]             # next turn of an earlier conversation
            prompt = base + [int(x) for x in rng.integers(0, 50000, int(rng.integers(5, 400)))]
        elif rng.random() < 0.7:
            prompt = system + [int(x) for x in rng.integers(0, 50000, int(rng.integers(1, 900)))]
        else:
            prompt = [int(x) for x in rng.integers(0, 50000, int(rng.integers(2, 1500)))]
        live, reuse = 0, 0
        start, valid = store.restore(0, None, prompt, live, reuse)
        want_start, _, _ = orc.restore(prompt, live, reuse)
        assert start == want_start, f"step {step}"
        ring_valid_from = 0 if start is None else valid
        if start is not None:
            assert valid == start - 128
        reply = [int(x) for x in rng.integers(0, 50000, int(rng.integers(1, 300)))]
        seq = prompt + reply
        position = len(seq) - int(rng.integers(0, 2))
        ends = [len(prompt), len(seq)]
        store.save(0, None, seq, position, ends, ring_valid_from)
        orc.save(seq, position, ends, ring_valid_from)
        convs.append(seq)
        _same_state(store, orc, [seq, prompt, system] + convs[-3:])
        assert store.stats()["bytes"] <= limit
    assert orc.evicted > 0, "the trace must exercise eviction"
    store.remove_all()
    assert store.stats()["blocks"] == 0 and store.stats()["bytes"] == 0
    store.close()


def test_checkpoint_only_where_the_ring_still_holds_it():
    # a long sequence: the turn checkpoint far behind the end is outside the ring and is skipped
    rng = np.random.default_rng(2)
    store, orc = _store(10 ** 9, ring=1024), po.PrefixOracle(10 ** 9, FULL, WIN, ring=1024)
    seq = [int(x) for x in rng.integers(0, 1000, 5000)]
    for ends in ([600, 5000], [3000, 4990], [200]):
        store.save(0, None, seq, 5000, ends, 0)
        orc.save(seq, 5000, ends, 0)
        _same_state(store, orc, [seq])
    wins = [i for i, (_, w) in enumerate(store.chain(seq)) if w]
    assert wins == [b.index for b in orc.chain(seq, 5000) if b.window] and 37 in wins and 3 not in wins
    # a restored sequence does not checkpoint blocks before the restore point
    store.save(0, None, seq, 5000, [4500], 4480)
    orc.save(seq, 5000, [4500], 4480)
    _same_state(store, orc, [seq])
    store.close()


def test_limit_zero_stores_nothing_and_bad_arguments():
    from embla_metal_b200 import attn
    store = _store(0)
    store.save(0, None, list(range(1000)), 1000, [1000], 0)
    assert store.stats()["blocks"] == 0
    assert store.restore(0, None, list(range(1000))) == (None, None)
    store.close()
    import pytest
    with pytest.raises(attn.EmblaError):
        _store(-1)
