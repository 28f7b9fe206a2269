"""TEST INFRASTRUCTURE - CPU restatement of the reference's prefix store index, used only by tests/ to check the
native store's decisions (which blocks are stored, checkpointed, evicted, where a prompt resumes).

Follows Sources/EmblaMetal/PrefixCache.swift: Block (:33-55), hash (:69-79), chain (:82-96), touch (:99-102),
insert (:105-114), addWindow (:116-119), evict (:124-131), remove (:138-144), Engine.restoreFromStore (:218-241) and
Engine.saveToStore (:247-285). No data is held: a block's buffers are byte counts. PARITY UNPINNED: the reference's
tests hold no vectors for the store; `embla-bench cache` (Sources/EmblaBench/Cache.swift:60-69) checks that a hit
reproduces the from-scratch run bit for bit, which the GPU test restates.

Among blocks of equal age the reference evicts in dictionary order (unspecified); this restatement and the native
store both take the lowest hash.
"""

BLOCK, TURN_MARGIN = 128, 16
MASK = (1 << 64) - 1


def fnv_hash(parent, tokens):
    h = (parent ^ 0xCBF29CE484222325) & MASK
    for t in tokens:
        v = t & 0xFFFFFFFF
        for _ in range(4):
            h = ((h ^ (v & 0xFF)) * 0x100000001B3) & MASK
            v >>= 8
    return h


class Block:
    def __init__(self, h, parent, index, tokens):
        self.hash, self.parent, self.index, self.tokens = h, parent, index, list(tokens)
        self.window = False
        self.children = 0
        self.last_use = 0

    @property
    def end(self):
        return (self.index + 1) * BLOCK


class PrefixOracle:
    def __init__(self, limit, full_bytes, window_bytes, ring=4096, turn_margin=TURN_MARGIN):
        self.limit, self.full_bytes, self.window_bytes, self.ring, self.turn_margin = limit, full_bytes, window_bytes, ring, turn_margin
        self.blocks = {}
        self.clock = 0
        self.bytes = 0
        self.evicted = 0

    def _bytes(self, b):
        return self.full_bytes + (self.window_bytes if b.window else 0)

    def chain(self, tokens, up_to):
        out, parent, j = [], None, 0
        while (j + 1) * BLOCK <= up_to:
            sl = list(tokens[j * BLOCK:(j + 1) * BLOCK])
            h = fnv_hash(parent.hash if parent else 0, sl)
            b = self.blocks.get(h)
            if b is None or b.parent is not parent or b.index != j or b.tokens != sl:
                break
            out.append(b)
            parent = b
            j += 1
        return out

    def touch(self, chain):
        self.clock += 1
        for b in chain:
            b.last_use = self.clock

    def _remove(self, b):
        del self.blocks[b.hash]
        self.bytes -= self._bytes(b)
        self.evicted += 1
        if b.parent is None:
            return
        b.parent.children -= 1
        if b.parent.children == 0 and not b.parent.window:
            self._remove(b.parent)

    def evict(self, keep=()):
        while self.bytes > self.limit:
            cands = [b for b in self.blocks.values() if b.children == 0 and b.hash not in keep]
            if not cands:
                return
            self._remove(min(cands, key=lambda b: (b.last_use, b.hash)))

    def restore(self, prompt, live, reuse):
        """(start, copied block indices, checkpoint block index) or (None, [], None)."""
        if self.limit <= 0:
            return None, [], None
        chain = self.chain(prompt, len(prompt) - 1)
        ks = [i for i, b in enumerate(chain) if b.window]
        if not ks or chain[ks[-1]].end <= reuse:
            self.touch(chain)
            return None, [], None
        k = ks[-1]
        used = chain[:k + 1]
        self.touch(used)
        return used[k].end, [b.index for b in used if b.end > live], used[k].index

    def save(self, tokens, position, turn_ends, ring_valid_from=0):
        """Returns (new block indices, new checkpoint indices)."""
        if self.limit <= 0:
            return [], []
        wanted = {(e - self.turn_margin) // BLOCK - 1 for e in turn_ends if e - self.turn_margin >= BLOCK}
        chain = self.chain(tokens, position)
        new_blocks, new_windows = [], []
        j = len(chain)
        while (j + 1) * BLOCK <= position:
            parent = chain[-1] if chain else None
            sl = list(tokens[j * BLOCK:(j + 1) * BLOCK])
            h = fnv_hash(parent.hash if parent else 0, sl)
            if h in self.blocks:
                break
            b = Block(h, parent, j, sl)
            b.last_use = self.clock
            self.blocks[h] = b
            if parent:
                parent.children += 1
            self.bytes += self.full_bytes
            chain.append(b)
            new_blocks.append(j)
            j += 1
        for b in chain:
            if b.window:
                continue
            p0 = b.index * BLOCK
            if p0 < ring_valid_from or position - p0 > self.ring or b.index not in wanted:
                continue
            b.window = True
            self.bytes += self.window_bytes
            new_windows.append(b.index)
        self.touch(chain)
        self.evict(keep={b.hash for b in chain})
        if self.bytes > self.limit:
            self.evict()
        return new_blocks, new_windows
