"""Host-side mirror of the reference's prefix store (PrefixCache, Sources/EmblaMetal/PrefixCache.swift:24-145;
Engine.restoreFromStore / saveToStore, PrefixCache.swift:218-285) over the native store of the CUDA library.

    store = PrefixStore(limit_bytes, pool=pool, rings=[ring, ...], n_kv_heads=4)
    store.save(seq, block_ids, tokens, position, turn_ends, ring_valid_from)
    start, ring_valid_from = store.restore(seq, block_ids, prompt, live, reuse)      # start None: no hit

`dry_run=True` (or no pool) keeps the index only: no device memory, no copies; it runs without a GPU.
"""
import ctypes as C

import numpy as np

from . import attn

BLOCK = 128          # PrefixCache.block
TURN_MARGIN = 16     # PrefixCache.turnMargin


class PrefixConfig(C.Structure):
    _fields_ = [("limit_bytes", C.c_int64), ("turn_margin", C.c_int32), ("dry_run", C.c_int32)]


class SeqCaches(C.Structure):
    _fields_ = [("pool", C.c_void_p), ("block_table_host", C.c_void_p), ("table_len", C.c_int32), ("rings", C.c_void_p),
                ("n_rings", C.c_int32), ("n_kv_heads", C.c_int32), ("ring_slots", C.c_int32), ("seq", C.c_int32)]


def _lib():
    L = attn.lib()
    L.embla_prefix_hash.restype = C.c_uint64
    L.embla_prefix_hash.argtypes = [C.c_uint64, C.c_void_p, C.c_int32]
    L.embla_prefix_store_destroy.argtypes = [C.c_void_p]
    L.embla_prefix_store_remove_all.argtypes = [C.c_void_p]
    L.embla_prefix_store_chain.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_int32]
    return L


def _tokens(tokens):
    return np.ascontiguousarray(np.asarray(tokens, dtype=np.int32))


def prefix_hash(parent, tokens):
    """FNV-1a over the tokens' bytes, started from the parent block's hash (PrefixCache.swift:69-79)."""
    t = _tokens(tokens)
    return int(_lib().embla_prefix_hash(C.c_uint64(parent), t.ctypes.data, len(t)))


class PrefixStore:
    def __init__(self, limit_bytes, pool=None, rings=(), n_kv_heads=4, ring_slots=4096, turn_margin=TURN_MARGIN, dry_run=False,
                 full_block_bytes=None, window_bytes=None):
        self.pool, self.rings, self.n_kv_heads = pool, list(rings), n_kv_heads
        self.dry_run = bool(dry_run or pool is None)
        self.ring_slots = self.rings[0].desc.ring if self.rings else ring_slots
        if full_block_bytes is None:
            full_block_bytes = pool.block_bytes
        if window_bytes is None:
            window_bytes = len(self.rings) * 2 * n_kv_heads * BLOCK * 256
        self.full_block_bytes, self.window_bytes = full_block_bytes, window_bytes
        self._ring_descs = (attn.RingDesc * max(1, len(self.rings)))(*[r.desc for r in self.rings])
        cfg = PrefixConfig(limit_bytes, turn_margin, int(self.dry_run))
        self.handle = C.c_void_p()
        attn._check(_lib().embla_prefix_store_create(C.byref(cfg), C.c_int64(full_block_bytes), C.c_int64(window_bytes),
                                                     C.byref(self.handle)))

    def close(self):
        if self.handle:
            _lib().embla_prefix_store_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:   # interpreter shutdown
            pass

    def remove_all(self):
        _lib().embla_prefix_store_remove_all(self.handle)

    def stats(self):
        b, n, cp, ev = C.c_int64(), C.c_int32(), C.c_int32(), C.c_int64()
        attn._check(_lib().embla_prefix_store_stats(self.handle, C.byref(b), C.byref(n), C.byref(cp), C.byref(ev)))
        return {"bytes": b.value, "blocks": n.value, "checkpoints": cp.value, "evicted": ev.value}

    def chain(self, tokens, up_to=None):
        """[(hash, has_checkpoint)] of the stored blocks `tokens` starts with (PrefixCache.chain)."""
        t = _tokens(tokens)
        up_to = len(t) if up_to is None else up_to
        cap = len(t) // BLOCK + 1
        hashes, wins = np.zeros(cap, np.uint64), np.zeros(cap, np.int32)
        n = _lib().embla_prefix_store_chain(self.handle, t.ctypes.data, len(t), up_to, hashes.ctypes.data, wins.ctypes.data, cap)
        return [(int(hashes[i]), bool(wins[i])) for i in range(n)]

    def _caches(self, seq, block_ids):
        table = np.ascontiguousarray(np.asarray(block_ids if block_ids is not None else [], dtype=np.int32))
        c = SeqCaches(None if self.dry_run else self.pool.handle, table.ctypes.data, len(table),
                      C.cast(self._ring_descs, C.c_void_p), len(self.rings), self.n_kv_heads, self.ring_slots, seq)
        return c, table   # the table must outlive the call

    def _stream(self):
        return None if self.dry_run else attn._stream()

    def restore(self, seq, block_ids, prompt, live=0, reuse=0):
        """(start, ring_valid_from), or (None, None) when the store does not beat `reuse`."""
        t = _tokens(prompt)
        c, _keep = self._caches(seq, block_ids)
        start, valid = C.c_int32(-1), C.c_int32(0)
        attn._check(_lib().embla_prefix_store_restore(self.handle, C.byref(c), C.c_void_p(t.ctypes.data), len(t), live, reuse, C.byref(start),
                                                      C.byref(valid), self._stream()))
        return (None, None) if start.value < 0 else (start.value, valid.value)

    def save(self, seq, block_ids, tokens, position, turn_ends, ring_valid_from=0):
        t = _tokens(tokens)
        ends = _tokens(turn_ends)
        c, _keep = self._caches(seq, block_ids)
        attn._check(_lib().embla_prefix_store_save(self.handle, C.byref(c), C.c_void_p(t.ctypes.data), position, C.c_void_p(ends.ctypes.data), len(ends),
                                                   ring_valid_from, self._stream()))
