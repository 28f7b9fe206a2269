// One decode step of attention through a stack of layers: the attention half of the reference's
// Engine.encodeStep / encodeAttention loop (Sources/EmblaMetal/Engine.swift:743-832, 933-991) as
// native host code, so that a step is one C call enqueuing every kernel on the caller's stream.
// Layer kinds follow Embla.Kind (Engine.swift:14): sliding, full, sparse. A sparse layer here owns
// 16-bit keys and values and scores them itself (score -> select -> attend) once the sequence is
// past topk + recent keys; a full layer appends its quantised k, v and attends with ReLU².
#include <new>
#include <vector>

#include <cstdlib>

#include "common.cuh"

struct EmblaStack {
    EmblaAttn* ctx;
    std::vector<EmblaLayerDesc> layers;
    EmblaKVPool* full_pool;
    EmblaKVPool* sparse_pool;
    std::vector<EmblaRing> rings;
    float* scores;        // [max_batch][n_kv_heads][scores_ld]
    uint32_t* idx;        // [max_batch][n_kv_heads][1152]
    int scores_ld;
    // timing probe: events around every launch of one entry point
    int probe;            // entry point whose launches are timed (-1: none)
    int probe_first;      // 1: only the first such launch of a step call
    int probe_marks;      // events recorded by the current step call
    std::vector<cudaEvent_t> ev;
    int ev_used;
    int early_ok;         // launches may fetch their cache ahead of the preceding kernel (EMBLA_NO_EARLY=1 turns it off)
};

// What a launch of the step writes / streams, for the "early" rule: a launch may request its cache rows before the
// kernel ahead of it in the stream has finished only if that kernel writes none of them (it appends the current token
// to its own layer's cache, nothing else), and never as the first launch of a step (what ran before is not ours).
enum { TOUCH_NONE = -1, TOUCH_FULL = 1000, TOUCH_SPARSE = 2000, TOUCH_RING = 3000 };

using namespace embla;

extern "C" {

EmblaStatus embla_stack_create(EmblaAttn* ctx, const EmblaLayerDesc* layers, int32_t n_layers, EmblaKVPool* full_pool,
                               EmblaKVPool* sparse_pool, const EmblaRing* rings, int32_t n_rings, EmblaStack** out) {
    if (!ctx || !layers || n_layers <= 0 || !out) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_stack_create: null argument");
    *out = nullptr;
    for (int i = 0; i < n_layers; i++) {
        const EmblaLayerDesc& L = layers[i];
        if (L.kind == EMBLA_LAYER_FULL) {
            if (!full_pool || full_pool->kv_dtype != EMBLA_KV_INT8 || L.slot < 0 || L.slot >= full_pool->n_layers)
                EMBLA_FAIL(EMBLA_BAD_ARG, "embla_stack_create: layer %d (full) needs slot %d of an int8 pool", i, L.slot);
        } else if (L.kind == EMBLA_LAYER_SPARSE) {
            if (!sparse_pool || sparse_pool->kv_dtype != EMBLA_KV_16BIT || L.slot < 0 || L.slot >= sparse_pool->n_layers)
                EMBLA_FAIL(EMBLA_BAD_ARG, "embla_stack_create: layer %d (sparse) needs slot %d of a 16-bit pool", i, L.slot);
            if (L.g1_dev)
                EMBLA_FAIL(EMBLA_UNSUPPORTED, "embla_stack_create: layer %d: a sparse layer that scores its own keys takes "
                                              "its queries prenormed", i);
        } else if (L.kind == EMBLA_LAYER_SPARSE_SHARED) {
            if (!full_pool || full_pool->kv_dtype != EMBLA_KV_INT8 || L.slot < 0 || L.slot >= full_pool->n_layers)
                EMBLA_FAIL(EMBLA_BAD_ARG, "embla_stack_create: layer %d (sparse, shared cache) needs slot %d of an int8 pool", i, L.slot);
        } else if (L.kind == EMBLA_LAYER_SLIDING) {
            if (!rings || L.slot < 0 || L.slot >= n_rings)
                EMBLA_FAIL(EMBLA_BAD_ARG, "embla_stack_create: layer %d (sliding) needs ring %d of %d", i, L.slot, n_rings);
        } else {
            EMBLA_FAIL(EMBLA_BAD_ARG, "embla_stack_create: layer %d has kind %d", i, L.kind);
        }
    }
    bool selects = false;
    for (int i = 0; i < n_layers; i++)
        selects |= layers[i].kind == EMBLA_LAYER_SPARSE || layers[i].kind == EMBLA_LAYER_SPARSE_SHARED || layers[i].emit_scores != 0;
    if (selects && ctx->cfg.max_context > EMBLA_SELECT_MAX_KEYS)
        EMBLA_FAIL(EMBLA_UNSUPPORTED, "embla_stack_create: max_context %d is over the %d keys embla_select_keys ranks",
                   ctx->cfg.max_context, EMBLA_SELECT_MAX_KEYS);
    EmblaStack* st = new (std::nothrow) EmblaStack();
    if (!st) EMBLA_FAIL(EMBLA_OOM, "embla_stack_create: host allocation failed");
    st->ctx = ctx;
    st->layers.assign(layers, layers + n_layers);
    st->full_pool = full_pool;
    st->sparse_pool = sparse_pool;
    if (rings) st->rings.assign(rings, rings + n_rings);
    st->scores = nullptr;
    st->idx = nullptr;
    st->probe = -1;
    st->probe_first = 0;
    st->probe_marks = 0;
    st->ev_used = 0;
    {
        const char* e = getenv("EMBLA_NO_EARLY");
        st->early_ok = !(e && e[0] == '1');
    }
    st->scores_ld = (ctx->cfg.max_context + BLK - 1) / BLK * BLK;
    const size_t pairs = size_t(ctx->cfg.max_batch) * ctx->cfg.n_kv_heads;
    cudaError_t e = cudaSuccess;
    bool need_scores = sparse_pool != nullptr;
    for (int i = 0; i < n_layers; i++) need_scores |= layers[i].kind == EMBLA_LAYER_SPARSE_SHARED || layers[i].emit_scores != 0;
    if (need_scores) {
        e = cudaMalloc(&st->scores, pairs * st->scores_ld * sizeof(float));
        if (e == cudaSuccess) e = cudaMalloc(&st->idx, pairs * (EMBLA_TOPK + EMBLA_RECENT) * sizeof(uint32_t));
    }
    if (e != cudaSuccess) {
        cudaFree(st->scores);
        cudaFree(st->idx);
        delete st;
        set_error("embla_stack_create: scores/selection buffers: %s", cudaGetErrorString(e));
        return e == cudaErrorMemoryAllocation ? EMBLA_OOM : EMBLA_CUDA;
    }
    *out = st;
    return EMBLA_OK;
}

void embla_stack_destroy(EmblaStack* st) {
    if (!st) return;
    cudaFree(st->scores);
    cudaFree(st->idx);
    for (cudaEvent_t e : st->ev) cudaEventDestroy(e);
    delete st;
}

EmblaStatus embla_stack_set_probe(EmblaStack* st, int32_t entry) {
    if (!st) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_stack_set_probe: null stack");
    st->probe = entry < 0 ? -1 : (entry & 255);
    st->probe_first = entry >= 0 && (entry & EMBLA_PROBE_FIRST_ONLY) != 0;
    st->ev_used = 0;
    return EMBLA_OK;
}

EmblaStatus embla_stack_read_probe(EmblaStack* st, float* total_ms, int32_t* launches) {
    if (!st || !total_ms || !launches) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_stack_read_probe: null argument");
    float sum = 0.0f;
    for (int i = 0; i + 1 < st->ev_used; i += 2) {
        float ms = 0.0f;
        EMBLA_CUDA_TRY(cudaEventElapsedTime(&ms, st->ev[i], st->ev[i + 1]));
        sum += ms;
    }
    *total_ms = sum;
    *launches = st->ev_used / 2;
    st->ev_used = 0;
    return EMBLA_OK;
}

}  // extern "C"

static EmblaStatus probe_mark(EmblaStack* st, int entry, cudaStream_t s) {
    if (st->probe != entry || (st->probe_first && st->probe_marks >= 2)) return EMBLA_OK;
    st->probe_marks++;
    if (st->ev_used == int(st->ev.size())) {
        cudaEvent_t e;
        EMBLA_CUDA_TRY(cudaEventCreate(&e));
        st->ev.push_back(e);
    }
    EMBLA_CUDA_TRY(cudaEventRecord(st->ev[st->ev_used++], s));
    return EMBLA_OK;
}

// One launch of the step: `reads` is the cache it streams (TOUCH_*, for the early rule), `writes` the cache it appends to.
#define EMBLA_STEP(entry, reads, writes, call)                                                        \
    do {                                                                                              \
        if (EmblaStatus s_ = probe_mark(st, entry, s)) return s_;                                     \
        ctx->trace_tag = entry;                                                                       \
        ctx->pdl = use_pdl && last_write != -2; /* the step's first launch follows work that is not ours: plain order */ \
        ctx->early = st->early_ok && last_write != -2 && (reads) != TOUCH_NONE && last_write != (reads); \
        if (EmblaStatus s_ = (call)) return s_;                                                       \
        last_write = (writes);                                                                        \
        if (EmblaStatus s_ = probe_mark(st, entry, s)) return s_;                                     \
    } while (0)

extern "C" EmblaStatus embla_stack_decode_step(EmblaStack* st, const EmblaStackStep* step, void* stream) {
    if (!st) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_stack_decode_step: null argument");
    return embla_stack_decode_layers(st, step, 0, int32_t(st->layers.size()), stream);
}

extern "C" EmblaStatus embla_stack_decode_layers(EmblaStack* st, const EmblaStackStep* step, int32_t first_layer, int32_t n_layers,
                                                 void* stream) {
    if (!st || !step || !step->qkv_dev || !step->o_dev || !step->seq_lens_dev || !step->pos_dev)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_stack_decode_step: null argument");
    if (first_layer < 0 || n_layers < 0 || size_t(first_layer) + size_t(n_layers) > st->layers.size())
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_stack_decode_layers: layers %d .. %d of %d", first_layer, first_layer + n_layers,
                   int(st->layers.size()));
    EmblaAttn* ctx = st->ctx;
    const int Hq = ctx->cfg.n_q_heads, Hkv = ctx->cfg.n_kv_heads, B = step->batch;
    if (B <= 0 || B > ctx->cfg.max_batch) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_stack_decode_step: batch %d", B);
    const size_t esz = 2;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int max_len = step->max_seq_len > 0 ? step->max_seq_len : ctx->cfg.max_context;
    // The step's launches depend on one another in stream order only; with programmatic dependent launch each becomes
    // resident while the one before it drains (EMBLA_NO_PDL=1 in the environment turns it off).
    static const bool use_pdl = []() { const char* e = getenv("EMBLA_NO_PDL"); return !(e && e[0] == '1'); }();
    struct PdlScope {
        EmblaAttn* c;
        int old;
        PdlScope(EmblaAttn* c_, int v) : c(c_), old(c_->pdl) { c->pdl = v; }
        ~PdlScope() {
            c->pdl = old;
            c->early = 0;
            c->trace_tag = -1;
        }
    } pdl_scope(ctx, use_pdl ? 1 : 0);
    int last_write = -2;   // -2: nothing of this step launched yet
    st->probe_marks = 0;
    for (size_t li = size_t(first_layer); li < size_t(first_layer) + size_t(n_layers); li++) {
        const EmblaLayerDesc& L = st->layers[li];
        const uint8_t* row = static_cast<const uint8_t*>(step->qkv_dev) + li * step->qkv_layer_stride * esz;
        const void* qp = row;
        const void* kp = row + size_t(Hq) * HD * esz;
        const void* vp = row + size_t(Hq + Hkv) * HD * esz;
        void* op = static_cast<uint8_t*>(step->o_dev) + li * step->o_layer_stride * esz;
        EmblaQuery q;
        q.q_dev = qp;
        q.q_stride = step->qkv_stride;
        q.prenormed = L.g1_dev ? 0 : 1;
        q.ng = L.g1_dev ? (L.g2_dev ? 2 : 1) : 0;
        q.g1_dev = L.g1_dev;
        q.g2_dev = L.g2_dev;
        if (L.kind == EMBLA_LAYER_SLIDING) {
            const EmblaRing* ring = &st->rings[L.slot];
            // ring write + attention in one launch, as the reference's attn_sliding
            EMBLA_STEP(EMBLA_ENTRY_SLIDING_DECODE, TOUCH_RING + L.slot, TOUCH_RING + L.slot,
                       embla_attn_sliding_step(ctx, ring, step->seq_lens_dev, B, &q, kp, vp, step->qkv_stride, L.kgain_dev ? 0 : 1,
                                               L.kgain_dev, op, step->o_stride, stream));
            continue;
        }
        EmblaKVView view;
        view.batch = B;
        view.layer = L.slot;
        view.seq_lens_dev = step->seq_lens_dev;
        view.max_seq_len = max_len;
        if (L.kind == EMBLA_LAYER_FULL) {
            view.block_table_dev = step->full_table_dev;
            view.table_stride = step->full_table_stride;
            if (!view.block_table_dev) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_stack_decode_step: no block table for the full layers");
            // past topk + recent keys, a full layer followed by sparse layers that share its cache also scores
            // every key, and the selection runs right after it (Engine.swift:796-797, 819-827); the quantised append
            // of the current token (Engine.swift:756-762) rides in the same launch
            const bool scoring = L.emit_scores != 0 && max_len > EMBLA_TOPK + EMBLA_RECENT;
            EMBLA_STEP(EMBLA_ENTRY_FULL_DECODE, TOUCH_FULL + L.slot, TOUCH_FULL + L.slot,
                       embla_attn_full_step(ctx, st->full_pool, &view, &q, kp, vp, step->qkv_stride, L.norm_k, op, step->o_stride,
                                            scoring ? st->scores : nullptr, st->scores_ld, stream));
            if (scoring)
                EMBLA_STEP(EMBLA_ENTRY_SELECT, TOUCH_NONE, TOUCH_NONE,
                           embla_select_keys(ctx, st->scores, st->scores_ld, step->seq_lens_dev, B, max_len, st->idx, stream));
        } else if (L.kind == EMBLA_LAYER_SPARSE_SHARED) {
            // a sparse layer over the preceding full layer's int8 cache (Engine.swift:461-462): no KV of its own
            view.block_table_dev = step->full_table_dev;
            view.table_stride = step->full_table_stride;
            const bool selecting = max_len > EMBLA_TOPK + EMBLA_RECENT;
            EMBLA_STEP(EMBLA_ENTRY_SPARSE_DECODE, TOUCH_NONE, TOUCH_NONE,
                       embla_attn_sparse_decode_int8(ctx, st->full_pool, &view, &q, selecting ? st->idx : nullptr, op,
                                                     step->o_stride, stream));
        } else {
            view.block_table_dev = step->sparse_table_dev;
            view.table_stride = step->sparse_table_stride;
            if (!view.block_table_dev) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_stack_decode_step: no block table for the sparse layers");
            const bool selecting = max_len > EMBLA_TOPK + EMBLA_RECENT;   // Engine.swift:796
            if (selecting) {
                // the append of the current token rides in the scoring launch
                EMBLA_STEP(EMBLA_ENTRY_SCORE, TOUCH_SPARSE + L.slot, TOUCH_SPARSE + L.slot,
                           embla_score_keys_step(ctx, st->sparse_pool, &view, qp, step->qkv_stride, kp, vp, step->qkv_stride,
                                                 L.norm_k, st->scores, st->scores_ld, stream));
                EMBLA_STEP(EMBLA_ENTRY_SELECT, TOUCH_NONE, TOUCH_NONE,
                           embla_select_keys(ctx, st->scores, st->scores_ld, step->seq_lens_dev, B, max_len, st->idx, stream));
            } else {
                EMBLA_STEP(EMBLA_ENTRY_APPEND, TOUCH_NONE, TOUCH_SPARSE + L.slot,
                           embla_kv_append(ctx, st->sparse_pool, &view, step->pos_dev, 1, kp, vp, step->qkv_stride,
                                           step->qkv_stride, L.norm_k, stream));
            }
            EMBLA_STEP(EMBLA_ENTRY_SPARSE_DECODE, TOUCH_NONE, TOUCH_NONE,
                       embla_attn_sparse_decode(ctx, st->sparse_pool, &view, &q, selecting ? st->idx : nullptr, op,
                                                step->o_stride, stream));
        }
    }
    return EMBLA_OK;
}

// The attention branch of the reference's Prefill.encode loop (Sources/EmblaMetal/Prefill.swift:282-345) for a chunk of
// tokens: per layer the chunk's keys and values into the layer's cache, then the chunk's attention over it.
extern "C" EmblaStatus embla_stack_prefill_chunk(EmblaStack* st, const EmblaStackChunk* ck, void* stream) {
    if (!st || !ck || !ck->qkv_dev || !ck->o_dev || !ck->pos0_dev) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_stack_prefill_chunk: null argument");
    EmblaAttn* ctx = st->ctx;
    const int Hq = ctx->cfg.n_q_heads, Hkv = ctx->cfg.n_kv_heads, B = ck->batch, T = ck->n_tokens;
    const int n_layers = int(st->layers.size());
    if (B <= 0 || B > ctx->cfg.max_batch || T <= 0) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_stack_prefill_chunk: batch %d, n_tokens %d", B, T);
    if (ck->kv_only_layers < 0 || ck->kv_only_layers > n_layers)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_stack_prefill_chunk: %d K/V-only layers of %d", ck->kv_only_layers, n_layers);
    for (const EmblaLayerDesc& L : st->layers)
        if (L.kind == EMBLA_LAYER_SPARSE || L.kind == EMBLA_LAYER_SPARSE_SHARED)
            EMBLA_FAIL(EMBLA_UNSUPPORTED, "embla_stack_prefill_chunk: the stack has sparse layers (the reference's prefill half has none: "
                                          "their tokens go through embla_stack_decode_step)");
    const size_t esz = 2;
    const int max_len = ck->max_seq_len > 0 ? ck->max_seq_len : ctx->cfg.max_context;
    for (int li = 0; li < n_layers; li++) {
        const EmblaLayerDesc& L = st->layers[li];
        const bool kv_only = li >= n_layers - ck->kv_only_layers;
        const uint8_t* row = static_cast<const uint8_t*>(ck->qkv_dev) + size_t(li) * ck->qkv_layer_stride * esz;
        const void* kp = row + size_t(Hq) * HD * esz;
        const void* vp = row + size_t(Hq + Hkv) * HD * esz;
        void* op = static_cast<uint8_t*>(ck->o_dev) + size_t(li) * ck->o_layer_stride * esz;
        EmblaQuery q;
        q.q_dev = row;
        q.q_stride = ck->qkv_seq_stride;
        q.prenormed = L.g1_dev ? 0 : 1;
        q.g1_dev = L.g1_dev;
        q.g2_dev = L.g2_dev;
        if (L.kind == EMBLA_LAYER_SLIDING) {
            const EmblaRing* ring = &st->rings[L.slot];
            q.ng = L.g1_dev ? 1 : 0;
            if (EmblaStatus e = embla_sliding_write(ctx, ring, ck->pos0_dev, B, T, kp, vp, ck->qkv_token_stride, ck->qkv_seq_stride,
                                                    L.kgain_dev ? 0 : 1, L.kgain_dev, stream))
                return e;
            if (kv_only) continue;
            if (EmblaStatus e = embla_attn_sliding_prefill(ctx, ring, ck->pos0_dev, B, T, &q, ck->qkv_token_stride, op, ck->o_token_stride,
                                                           ck->o_seq_stride, stream))
                return e;
            continue;
        }
        if (!ck->full_table_dev) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_stack_prefill_chunk: no block table for the full layers");
        q.ng = L.g1_dev ? (L.g2_dev ? 2 : 1) : 0;
        EmblaKVView view;
        view.batch = B;
        view.layer = L.slot;
        view.seq_lens_dev = nullptr;
        view.max_seq_len = max_len;
        view.block_table_dev = ck->full_table_dev;
        view.table_stride = ck->full_table_stride;
        if (EmblaStatus e = embla_kv_append(ctx, st->full_pool, &view, ck->pos0_dev, T, kp, vp, ck->qkv_token_stride, ck->qkv_seq_stride,
                                            L.norm_k, stream))
            return e;
        if (kv_only) continue;
        if (EmblaStatus e = embla_attn_full_prefill(ctx, st->full_pool, &view, ck->pos0_dev, T, &q, ck->qkv_token_stride, op,
                                                    ck->o_token_stride, ck->o_seq_stride, stream))
            return e;
    }
    return EMBLA_OK;
}
