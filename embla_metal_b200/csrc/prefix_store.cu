// Prefix-cache store over the paged KV layout: keys and values of earlier sequences kept for prompts that
// start the same way. Replaces PrefixCache (Sources/EmblaMetal/PrefixCache.swift:24-145) and
// Engine.restoreFromStore / saveToStore with their span copies (PrefixCache.swift:150-286).
//
// The index is the reference's: sequences cut into blocks of 128 positions, a block known by an FNV-1a hash
// chained over its tokens and every token before it, a parent/child tree, window checkpoints only at turn
// ends, least-recently-used leaves evicted first. What differs is the data side. A stored block is ONE
// contiguous copy of a physical block of the pool (every full layer, K and V, every kv head, codes and scales:
// the reference blits about 40 spans); a checkpoint is the 128 ring slots of every sliding layer, gathered by one
// kernel launch into one buffer. Stored bytes live in slabs of device memory carved into two slot sizes, so a
// save or an eviction never calls the allocator once the slabs exist. The engram conv history the reference
// adds to a checkpoint is not part of this library (no engram here).
#include <algorithm>
#include <cstring>
#include <memory>
#include <set>
#include <unordered_map>
#include <vector>

#include "common.cuh"

namespace embla {

constexpr size_t PREFIX_SLAB_BYTES = size_t(64) << 20;

// Fixed-size slots carved from slabs; dry: no device memory, slots are distinct fake addresses.
struct SlotPool {
    size_t slot_bytes = 0;
    bool dry = false;
    std::vector<void*> slabs;
    std::vector<void*> free_slots;
    uintptr_t fake = 0x1000;

    void* take() {
        if (free_slots.empty()) {
            if (dry) {
                fake += 0x1000;
                return reinterpret_cast<void*>(fake);
            }
            const size_t per = std::max<size_t>(1, PREFIX_SLAB_BYTES / slot_bytes);
            void* slab = nullptr;
            if (cudaMalloc(&slab, per * slot_bytes) != cudaSuccess) {
                cudaGetLastError();
                return nullptr;
            }
            slabs.push_back(slab);
            for (size_t i = per; i-- > 0;) free_slots.push_back(static_cast<uint8_t*>(slab) + i * slot_bytes);
        }
        void* s = free_slots.back();
        free_slots.pop_back();
        return s;
    }
    void give(void* s) {
        if (s && !dry) free_slots.push_back(s);
    }
    void release_all() {
        for (void* s : slabs) cudaFree(s);
        slabs.clear();
        free_slots.clear();
    }
};

struct PrefixBlock {   // PrefixCache.Block (PrefixCache.swift:33-55)
    uint64_t hash;
    PrefixBlock* parent;
    int index;
    std::vector<int32_t> tokens;
    void* full;
    void* window = nullptr;
    int children = 0;
    uint64_t last_use = 0;
};

}  // namespace embla

struct EmblaPrefixStore {
    EmblaPrefixConfig cfg;
    int64_t full_bytes, window_bytes;
    embla::SlotPool full_slots, window_slots;
    std::unordered_map<uint64_t, std::unique_ptr<embla::PrefixBlock>> blocks;
    uint64_t clock = 0;
    int64_t bytes = 0;
    int64_t evicted = 0;

    int64_t bytes_of(const embla::PrefixBlock* b) const { return full_bytes + (b->window ? window_bytes : 0); }
};

namespace embla {

static uint64_t prefix_hash(uint64_t parent, const int32_t* tokens, int n) {   // PrefixCache.swift:69-79
    uint64_t h = parent ^ 0xcbf29ce484222325ull;
    for (int i = 0; i < n; i++) {
        uint32_t v = uint32_t(tokens[i]);
        for (int k = 0; k < 4; k++) {
            h = (h ^ uint64_t(v & 0xFF)) * 0x100000001b3ull;
            v >>= 8;
        }
    }
    return h;
}

// Walks the tree from the root along `tokens`, 128 at a time, while each next block is stored and ends inside the first
// `limit` positions; returns the blocks it passed (the lookup of PrefixCache.swift:82-96).
static std::vector<PrefixBlock*> chain_of(const EmblaPrefixStore* st, const int32_t* tokens, int limit) {
    std::vector<PrefixBlock*> out;
    PrefixBlock* parent = nullptr;
    int j = 0;
    while ((j + 1) * BLK <= limit) {
        const int32_t* slice = tokens + j * BLK;
        const uint64_t h = prefix_hash(parent ? parent->hash : 0, slice, BLK);
        auto it = st->blocks.find(h);
        if (it == st->blocks.end()) break;
        PrefixBlock* b = it->second.get();
        // a 64-bit hash can collide: the entry only counts if it hangs off the block we came from, at this depth, with
        // exactly these 128 tokens
        if (b->parent != parent || b->index != j || std::memcmp(b->tokens.data(), slice, BLK * sizeof(int32_t)) != 0) break;
        out.push_back(b);
        parent = b;
        j++;
    }
    return out;
}

static void touch(EmblaPrefixStore* st, const std::vector<PrefixBlock*>& chain) {   // PrefixCache.swift:99-102
    st->clock++;
    for (PrefixBlock* b : chain) b->last_use = st->clock;
}

static void remove_block(EmblaPrefixStore* st, PrefixBlock* b) {   // PrefixCache.swift:138-144
    PrefixBlock* parent = b->parent;
    st->bytes -= st->bytes_of(b);
    st->full_slots.give(b->full);
    st->window_slots.give(b->window);
    st->evicted++;
    st->blocks.erase(b->hash);
    if (!parent) return;
    parent->children--;
    if (parent->children == 0 && parent->window == nullptr) remove_block(st, parent);
}

// Over budget: leaves (blocks no stored block continues) are dropped oldest first until the bytes fit, sparing the
// hashes in `keep`; dropping a leaf can expose its parent as the next candidate (the policy of PrefixCache.swift:121-131).
// Among leaves of equal age the lower hash goes first, which makes the order reproducible (the reference walks a
// dictionary there, in no stated order).
static void evict(EmblaPrefixStore* st, const std::set<uint64_t>& keep) {
    while (st->bytes > st->cfg.limit_bytes) {
        PrefixBlock* lru = nullptr;
        for (auto& kv : st->blocks) {
            PrefixBlock* b = kv.second.get();
            if (b->children != 0 || keep.count(b->hash)) continue;
            if (!lru || b->last_use < lru->last_use || (b->last_use == lru->last_use && b->hash < lru->hash)) lru = b;
        }
        if (!lru) return;
        remove_block(st, lru);
    }
}

// ---- checkpoint copies: the 128 ring slots from p0 of every sliding layer, K then V, per kv head ------------
constexpr int PREFIX_MAX_RINGS = 48;
struct RingCopyParams {
    uint8_t* k[PREFIX_MAX_RINGS];
    uint8_t* v[PREFIX_MAX_RINGS];
    int64_t seq_off[PREFIX_MAX_RINGS];   // bytes from a ring's base to this sequence's rows
    uint8_t* stored;
    int n_kv_heads, ring, slot, save;
};

// grid (kv head, K|V, layer), 256 threads: one 32 KiB run of 128 slots x 256 B, 16 bytes per thread and trip.
__global__ void __launch_bounds__(256) ring_window_copy_kernel(const RingCopyParams p) {
    const int h = blockIdx.x, side = blockIdx.y, layer = blockIdx.z;
    uint8_t* ring = (side ? p.v[layer] : p.k[layer]) + p.seq_off[layer] + (size_t(h) * p.ring + p.slot) * (HD * 2);
    uint8_t* stored = p.stored + ((size_t(layer) * 2 + side) * p.n_kv_heads + h) * (BLK * HD * 2);
    const uint4* src = reinterpret_cast<const uint4*>(p.save ? ring : stored);
    uint4* dst = reinterpret_cast<uint4*>(p.save ? stored : ring);
    for (int i = threadIdx.x; i < BLK * HD * 2 / 16; i += blockDim.x) dst[i] = src[i];
}

static EmblaStatus copy_window(const EmblaSeqCaches* c, int p0, void* stored, bool save, cudaStream_t s) {
    if (c->n_rings > PREFIX_MAX_RINGS) EMBLA_FAIL(EMBLA_UNSUPPORTED, "prefix store: %d sliding layers (at most %d)", c->n_rings, PREFIX_MAX_RINGS);
    if (c->n_rings == 0) return EMBLA_OK;
    RingCopyParams p = {};
    for (int l = 0; l < c->n_rings; l++) {
        const EmblaRing& r = c->rings[l];
        if (r.ring != c->ring_slots || r.ring % BLK) EMBLA_FAIL(EMBLA_BAD_ARG, "prefix store: ring of %d slots (want %d, a multiple of 128)", r.ring, c->ring_slots);
        p.k[l] = static_cast<uint8_t*>(r.k_dev);
        p.v[l] = static_cast<uint8_t*>(r.v_dev);
        p.seq_off[l] = int64_t(c->seq) * r.seq_stride * 2;
    }
    p.stored = static_cast<uint8_t*>(stored);
    p.n_kv_heads = c->n_kv_heads;
    p.ring = c->ring_slots;
    p.slot = p0 % c->ring_slots;
    p.save = save;
    ring_window_copy_kernel<<<dim3(c->n_kv_heads, 2, c->n_rings), 256, 0, s>>>(p);
    EMBLA_CUDA_TRY(cudaGetLastError());
    return EMBLA_OK;
}

static EmblaStatus copy_full(const EmblaSeqCaches* c, int index, void* stored, bool save, cudaStream_t s) {
    if (index >= c->table_len) EMBLA_FAIL(EMBLA_BAD_ARG, "prefix store: block %d beyond the block table (%d entries)", index, c->table_len);
    const int id = c->block_table_host[index];
    if (id < 0 || id >= c->pool->num_blocks) EMBLA_FAIL(EMBLA_BAD_ARG, "prefix store: physical block %d outside the pool", id);
    uint8_t* at = c->pool->base + size_t(id) * c->pool->block_bytes;
    EMBLA_CUDA_TRY(cudaMemcpyAsync(save ? stored : at, save ? at : stored, c->pool->block_bytes, cudaMemcpyDeviceToDevice, s));
    return EMBLA_OK;
}

static EmblaStatus check_caches(const EmblaPrefixStore* st, const EmblaSeqCaches* c, const char* fn) {
    if (!c) EMBLA_FAIL(EMBLA_BAD_ARG, "%s: null caches", fn);
    if (c->ring_slots <= 0 || c->ring_slots % BLK) EMBLA_FAIL(EMBLA_BAD_ARG, "%s: ring_slots %d must be a positive multiple of 128", fn, c->ring_slots);
    if (st->cfg.dry_run) return EMBLA_OK;
    if (!c->pool || !c->block_table_host || (c->n_rings > 0 && !c->rings)) EMBLA_FAIL(EMBLA_BAD_ARG, "%s: null pool, block table or rings", fn);
    if (int64_t(c->pool->block_bytes) != st->full_bytes)
        EMBLA_FAIL(EMBLA_BAD_ARG, "%s: the pool's blocks hold %zu bytes, the store's %lld", fn, c->pool->block_bytes, (long long)st->full_bytes);
    if (int64_t(c->n_rings) * 2 * c->n_kv_heads * BLK * HD * 2 != st->window_bytes)
        EMBLA_FAIL(EMBLA_BAD_ARG, "%s: %d rings x %d kv heads do not match the store's checkpoints of %lld bytes", fn, c->n_rings,
                   c->n_kv_heads, (long long)st->window_bytes);
    return EMBLA_OK;
}

}  // namespace embla

using namespace embla;

extern "C" {

uint64_t embla_prefix_hash(uint64_t parent, const int32_t* tokens, int32_t n) { return prefix_hash(parent, tokens, n); }

EmblaStatus embla_prefix_store_create(const EmblaPrefixConfig* cfg, int64_t full_block_bytes, int64_t window_bytes,
                                      EmblaPrefixStore** out) {
    if (!cfg || !out) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_prefix_store_create: null argument");
    *out = nullptr;
    if (cfg->limit_bytes < 0 || cfg->turn_margin < 0 || full_block_bytes <= 0 || window_bytes < 0)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_prefix_store_create: limit %lld, margin %d, block %lld, checkpoint %lld bytes",
                   (long long)cfg->limit_bytes, cfg->turn_margin, (long long)full_block_bytes, (long long)window_bytes);
    EmblaPrefixStore* st = new EmblaPrefixStore();
    st->cfg = *cfg;
    st->full_bytes = full_block_bytes;
    st->window_bytes = window_bytes;
    st->full_slots.slot_bytes = size_t(full_block_bytes);
    st->window_slots.slot_bytes = size_t(std::max<int64_t>(window_bytes, 16));
    st->full_slots.dry = st->window_slots.dry = cfg->dry_run != 0;
    *out = st;
    return EMBLA_OK;
}

void embla_prefix_store_remove_all(EmblaPrefixStore* st) {   // PrefixCache.swift:133-136
    if (!st) return;
    for (auto& kv : st->blocks) {
        st->full_slots.give(kv.second->full);
        st->window_slots.give(kv.second->window);
    }
    st->blocks.clear();
    st->bytes = 0;
}

void embla_prefix_store_destroy(EmblaPrefixStore* st) {
    if (!st) return;
    embla_prefix_store_remove_all(st);
    st->full_slots.release_all();
    st->window_slots.release_all();
    delete st;
}

EmblaStatus embla_prefix_store_stats(const EmblaPrefixStore* st, int64_t* bytes, int32_t* blocks, int32_t* checkpoints,
                                     int64_t* evicted) {
    if (!st) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_prefix_store_stats: null store");
    int32_t cp = 0;
    for (auto& kv : st->blocks) cp += kv.second->window != nullptr;
    if (bytes) *bytes = st->bytes;
    if (blocks) *blocks = int32_t(st->blocks.size());
    if (checkpoints) *checkpoints = cp;
    if (evicted) *evicted = st->evicted;
    return EMBLA_OK;
}

int32_t embla_prefix_store_chain(const EmblaPrefixStore* st, const int32_t* tokens, int32_t n_tokens, int32_t up_to,
                                 uint64_t* hashes_out, int32_t* has_window_out, int32_t cap) {
    if (!st || !tokens) return -1;
    const std::vector<PrefixBlock*> chain = chain_of(st, tokens, std::min(up_to, n_tokens));
    for (size_t i = 0; i < chain.size() && int32_t(i) < cap; i++) {
        if (hashes_out) hashes_out[i] = chain[i]->hash;
        if (has_window_out) has_window_out[i] = chain[i]->window != nullptr;
    }
    return int32_t(chain.size());
}

// Engine.restoreFromStore (PrefixCache.swift:218-241)
EmblaStatus embla_prefix_store_restore(EmblaPrefixStore* st, const EmblaSeqCaches* dst, const int32_t* prompt, int32_t n_prompt,
                                       int32_t live, int32_t reuse, int32_t* start_out, int32_t* ring_valid_from_out,
                                       void* stream) {
    if (!st || !prompt || !start_out) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_prefix_store_restore: null argument");
    *start_out = -1;
    if (st->cfg.limit_bytes <= 0) return EMBLA_OK;
    if (EmblaStatus e = check_caches(st, dst, "embla_prefix_store_restore")) return e;
    const std::vector<PrefixBlock*> chain = chain_of(st, prompt, n_prompt - 1);
    int k = -1;
    for (int i = int(chain.size()) - 1; i >= 0; i--)
        if (chain[i]->window) {
            k = i;
            break;
        }
    if (k < 0 || (chain[k]->index + 1) * BLK <= reuse) {
        touch(st, chain);
        return EMBLA_OK;
    }
    const std::vector<PrefixBlock*> used(chain.begin(), chain.begin() + k + 1);
    touch(st, used);
    const int start = (used[k]->index + 1) * BLK;
    if (!st->cfg.dry_run) {
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        // the blocks the live caches lack (they hold positions before `live`), then the checkpoint
        for (PrefixBlock* b : used)
            if ((b->index + 1) * BLK > live)
                if (EmblaStatus e = copy_full(dst, b->index, b->full, false, s)) return e;
        if (EmblaStatus e = copy_window(dst, used[k]->index * BLK, used[k]->window, false, s)) return e;
    }
    *start_out = start;
    if (ring_valid_from_out) *ring_valid_from_out = start - BLK;   // the rings hold this sequence from the checkpoint on
    return EMBLA_OK;
}

// Engine.saveToStore (PrefixCache.swift:247-285)
EmblaStatus embla_prefix_store_save(EmblaPrefixStore* st, const EmblaSeqCaches* src, const int32_t* tokens, int32_t position,
                                    const int32_t* turn_ends, int32_t n_turn_ends, int32_t ring_valid_from, void* stream) {
    if (!st || !tokens || (n_turn_ends > 0 && !turn_ends)) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_prefix_store_save: null argument");
    if (st->cfg.limit_bytes <= 0) return EMBLA_OK;
    if (EmblaStatus e = check_caches(st, src, "embla_prefix_store_save")) return e;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    std::set<int> wanted;   // block indices to checkpoint
    for (int i = 0; i < n_turn_ends; i++)
        if (turn_ends[i] - st->cfg.turn_margin >= BLK) wanted.insert((turn_ends[i] - st->cfg.turn_margin) / BLK - 1);
    std::vector<PrefixBlock*> chain = chain_of(st, tokens, position);
    int j = int(chain.size());
    while ((j + 1) * BLK <= position) {
        PrefixBlock* parent = chain.empty() ? nullptr : chain.back();
        const uint64_t h = prefix_hash(parent ? parent->hash : 0, tokens + j * BLK, BLK);
        if (st->blocks.count(h)) break;   // stored for other tokens
        void* slot = st->full_slots.take();
        if (!slot) break;
        if (!st->cfg.dry_run)
            if (EmblaStatus e = copy_full(src, j, slot, true, s)) {
                st->full_slots.give(slot);
                return e;
            }
        auto b = std::make_unique<PrefixBlock>();
        b->hash = h;
        b->parent = parent;
        b->index = j;
        b->tokens.assign(tokens + j * BLK, tokens + (j + 1) * BLK);
        b->full = slot;
        b->last_use = st->clock;
        if (parent) parent->children++;
        st->bytes += st->full_bytes;
        chain.push_back(b.get());
        st->blocks[h] = std::move(b);
        j++;
    }
    for (PrefixBlock* b : chain) {
        if (b->window) continue;
        const int p0 = b->index * BLK;
        // a checkpoint we keep, whose ring slots hold this sequence's positions (not overwritten since, nor left
        // from another sequence by a restore)
        if (p0 < ring_valid_from || position - p0 > src->ring_slots || !wanted.count(b->index)) continue;
        void* slot = st->window_slots.take();
        if (!slot) continue;
        if (!st->cfg.dry_run)
            if (EmblaStatus e = copy_window(src, p0, slot, true, s)) {
                st->window_slots.give(slot);
                return e;
            }
        b->window = slot;
        st->bytes += st->window_bytes;
    }
    touch(st, chain);
    std::set<uint64_t> keep;
    for (PrefixBlock* b : chain) keep.insert(b->hash);
    evict(st, keep);
    if (st->bytes > st->cfg.limit_bytes) evict(st, {});
    // An evicted slot may be handed out again by the next save: its copy is ordered after these on `stream`.
    return EMBLA_OK;
}

}  // extern "C"
