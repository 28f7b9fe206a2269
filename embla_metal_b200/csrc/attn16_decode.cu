// Softmax decode attention over 16-bit keys and values, one query token per sequence:
//  * sparse layers (Sources/EmblaMetal/Kernels/attention.metal:370-441, 448-584, 593-645; dispatch
//    Sources/EmblaMetal/Engine.swift:796-818): every key while the sequence has at most 1152, else
//    the 1152 selected rows idx[kv head][..] gathered from the paged pool;
//  * sliding layers (attention.metal:26-102): the last `window` positions of a ring, after the
//    ring write of the current token (sliding_write_kernel; attention.metal:47-62 and
//    kv_sliding_b, Sources/EmblaMetal/Kernels/prefill.metal:105-125).
//
// The kernel (attn16_kernel.cuh) streams 64-row tiles of one (sequence, kv head) through a cp.async ring
// with an online softmax; a pair's rows are cut into as many ranges as fill the device, merged through
// (max, sum, acc) partials by the last CTA to arrive, in range order (attention.metal:428-440).
#include <cstdlib>

#include "attn16_kernel.cuh"

namespace embla {

// ---- ring write of the sliding layers -------------------------------------------------------------
struct SlidingWriteParams {
    const void* k;
    const void* v;
    const void* kg;
    uint8_t* ring_k;
    uint8_t* ring_v;
    const int32_t* pos0;
    int64_t token_stride, seq_stride, ring_stride;
    int batch, n_tokens, n_kv_heads, ring, prenormed;
    float rope_freq[32];
};

template <int DT>
__global__ void __launch_bounds__(128) sliding_write_kernel(const SlidingWriteParams p) {
    const int lane = threadIdx.x & 31;
    const long warp = (long(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const long total = long(p.batch) * p.n_tokens * p.n_kv_heads;
    if (warp >= total) return;
    const int h = int(warp % p.n_kv_heads);
    const long bt = warp / p.n_kv_heads;
    const int t = int(bt % p.n_tokens), b = int(bt / p.n_tokens);
    const int pos = p.pos0[b] + t, slot = pos % p.ring;
    const size_t off = size_t(b) * p.seq_stride + size_t(t) * p.token_stride + size_t(h) * HD;
    float x[4];
#pragma unroll
    for (int i = 0; i < 4; i++) x[i] = Act<DT>::load(p.k, off + lane + 32 * i);
    if (!p.prenormed) norm_rope_round<DT>(x, p.kg, p.kg, 1, pos, p.rope_freq, lane);
    const size_t dst = size_t(b) * p.ring_stride + (size_t(h) * p.ring + slot) * HD;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        Act<DT>::store(p.ring_k, dst + lane + 32 * i, x[i]);
        reinterpret_cast<uint16_t*>(p.ring_v)[dst + lane + 32 * i] =
            reinterpret_cast<const uint16_t*>(p.v)[off + lane + 32 * i];
    }
}

}  // namespace embla

using namespace embla;

static EmblaStatus check_query(const char* fn, const EmblaQuery* q) {
    if (!q || !q->q_dev) EMBLA_FAIL(EMBLA_BAD_ARG, "%s: null query", fn);
    if (!q->prenormed && (q->ng < 0 || q->ng > 2 || (q->ng >= 1 && !q->g1_dev) || (q->ng >= 2 && !q->g2_dev)))
        EMBLA_FAIL(EMBLA_BAD_ARG, "%s: ng %d without its gain vectors", fn, q->ng);
    return EMBLA_OK;
}

// Tensor maps over a sliding layer's K and V rings for the ring-tile path: bytes [sequence][kv head x slot][256], boxes of
// 64 rows x 128 bytes under the 128-byte swizzle. Encoded once per (ring, batch) and kept in the context.
static EmblaStatus ring_maps(EmblaAttn* ctx, const Attn16Params& p, int batch, const CUtensorMap** mk, const CUtensorMap** mv) {
    for (int i = 0; i < ctx->ring_maps_used; i++) {
        const EmblaAttn::RingMaps& m = ctx->ring_maps[i];
        if (m.k == p.ring_k && m.v == p.ring_v && m.seq_stride == p.ring_stride && m.ring == p.ring &&
            m.n_kv_heads == p.n_kv_heads && m.batch == batch) {
            *mk = &m.mk;
            *mv = &m.mv;
            return EMBLA_OK;
        }
    }
    TensorMapEncodeTiledFn enc = tensor_map_encoder();
    if (!enc) EMBLA_FAIL(EMBLA_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    EmblaAttn::RingMaps& m = ctx->ring_maps[ctx->ring_maps_next];
    const cuuint64_t dims[3] = {HD * 2, cuuint64_t(p.n_kv_heads) * p.ring, cuuint64_t(batch)};
    const cuuint64_t strides[2] = {HD * 2, cuuint64_t(p.ring_stride) * 2};
    const cuuint32_t box[3] = {128, A16_ROWS, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    for (int side = 0; side < 2; side++) {
        CUresult r = enc(side ? &m.mv : &m.mk, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<uint8_t*>(side ? p.ring_v : p.ring_k), dims,
                         strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) {
            m.k = nullptr;
            EMBLA_FAIL(EMBLA_CUDA, "cuTensorMapEncodeTiled failed for a ring (%d)", int(r));
        }
    }
    m.k = p.ring_k;
    m.v = p.ring_v;
    m.seq_stride = p.ring_stride;
    m.ring = p.ring;
    m.n_kv_heads = p.n_kv_heads;
    m.batch = batch;
    ctx->ring_maps_next = (ctx->ring_maps_next + 1) % EmblaAttn::RING_MAP_SLOTS;
    if (ctx->ring_maps_used < EmblaAttn::RING_MAP_SLOTS) ctx->ring_maps_used++;
    *mk = &m.mk;
    *mv = &m.mv;
    return EMBLA_OK;
}

template <int DT, int MODE, bool TMA, bool CL>
static EmblaStatus launch_attn16_kernel(EmblaAttn* ctx, const Attn16Params& p, const CUtensorMap& mk, const CUtensorMap& mv,
                                        dim3 grid, cudaStream_t s) {
    constexpr size_t smem = 1024 + A16_STAGES * A16_STAGE + 8 * HD * 2 + (CL ? A16_INBOX_BYTES : 0);
    static bool configured[64] = {};
    if (!configured[ctx->device & 63]) {
        EMBLA_CUDA_TRY(cudaFuncSetAttribute(attn16_decode_kernel<DT, MODE, TMA, CL>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        configured[ctx->device & 63] = true;
    }
    EMBLA_CUDA_TRY(launch_kernel_cluster(ctx->pdl, CL ? int(grid.x) : 1, attn16_decode_kernel<DT, MODE, TMA, CL>, grid,
                                         dim3(A16_THREADS + (TMA ? 32 : 0)), smem, s, p, mk, mv));
    EMBLA_CUDA_TRY(cudaGetLastError());
    return EMBLA_OK;
}

template <int DT, int MODE, bool TMA>
static EmblaStatus launch_attn16_cl(EmblaAttn* ctx, const Attn16Params& p, const CUtensorMap& mk, const CUtensorMap& mv, dim3 grid,
                                    bool cluster, cudaStream_t s) {
    return cluster ? launch_attn16_kernel<DT, MODE, TMA, true>(ctx, p, mk, mv, grid, s)
                   : launch_attn16_kernel<DT, MODE, TMA, false>(ctx, p, mk, mv, grid, s);
}

template <int MODE>
static EmblaStatus launch_attn16(EmblaAttn* ctx, Attn16Params& p, int batch, int max_rows, cudaStream_t s) {
    p.partials = ctx->partials;
    p.counters = ctx->counters;
    p.ctl = kernel_ctl(ctx);
    p.G = ctx->cfg.n_q_heads / ctx->cfg.n_kv_heads;
    p.n_kv_heads = ctx->cfg.n_kv_heads;
    // Rings of a multiple of 64 slots are read as tiles of 64 consecutive slots (TMA); the window then spans one tile
    // more unless it starts on a tile boundary.
    const bool tma = MODE == A16_SLIDING && p.ring % A16_ROWS == 0;
    // Ranges per pair: the count that minimises (waves of CTAs over 2 CTAs per SM) x (tiles of a range + the fixed cost
    // of a CTA in tiles: query set-up, pipeline fill, merge). Up to 8 ranges run as one thread-block cluster a pair and
    // merge through its shared memory (EMBLA_NO_CLUSTER=1: up to 16 ranges merged through global scratch by the last
    // CTA to arrive, the path that also serves when a cluster cannot be had).
    static const bool use_clusters = []() { const char* e = getenv("EMBLA_NO_CLUSTER"); return !(e && e[0] == '1'); }();
    const int ns_max = use_clusters ? 8 : 16;
    const int max_tiles = (max_rows > 0 ? (max_rows + A16_ROWS - 1) / A16_ROWS : 1) + (tma ? 1 : 0);
    const long pairs = long(batch) * p.n_kv_heads, slots = 2L * ctx->sm_count;
    long best_cost = -1;
    p.tiles_per_cta = max_tiles;
    p.max_chunks = 1;
    for (int ns = 1; ns <= ns_max && ns <= max_tiles; ns++) {
        const int tp = (max_tiles + ns - 1) / ns, nsr = (max_tiles + tp - 1) / tp;
        if (nsr > ns_max || (!use_clusters && pairs * nsr > ctx->partial_slots)) continue;
        const long waves = (pairs * nsr + slots - 1) / slots;
        const long cost = waves * (tp + 3 + (nsr > 1 ? 1 : 0));
        if (best_cost < 0 || cost < best_cost) {
            best_cost = cost;
            p.tiles_per_cta = tp;
            p.max_chunks = nsr;
        }
    }
    const bool cluster = use_clusters && p.max_chunks > 1;
    fill_rope_freq(p.rope_freq);
    dim3 grid(p.max_chunks, p.n_kv_heads, batch);
    const bool bf = ctx->cfg.act_dtype == EMBLA_BF16;
    if (tma) {
        const CUtensorMap *mk = nullptr, *mv = nullptr;
        if (EmblaStatus st = ring_maps(ctx, p, batch, &mk, &mv)) return st;
        return bf ? launch_attn16_cl<EMBLA_BF16, MODE, MODE == A16_SLIDING>(ctx, p, *mk, *mv, grid, cluster, s)
                  : launch_attn16_cl<EMBLA_F16, MODE, MODE == A16_SLIDING>(ctx, p, *mk, *mv, grid, cluster, s);
    }
    static const CUtensorMap none = {};
    return bf ? launch_attn16_cl<EMBLA_BF16, MODE, false>(ctx, p, none, none, grid, cluster, s)
              : launch_attn16_cl<EMBLA_F16, MODE, false>(ctx, p, none, none, grid, cluster, s);
}

extern "C" EmblaStatus embla_attn_sparse_decode(EmblaAttn* ctx, const EmblaKVPool* pool, const EmblaKVView* view,
                                                const EmblaQuery* q, const uint32_t* idx_dev, void* o_dev,
                                                int64_t o_stride, void* stream) {
    if (!ctx || !pool || !view || !o_dev) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_sparse_decode: null argument");
    EMBLA_CHECK_DEVICE("embla_attn_sparse_decode", ctx, pool);
    if (EmblaStatus st = check_query("embla_attn_sparse_decode", q)) return st;
    if (pool->kv_dtype != EMBLA_KV_16BIT)
        EMBLA_FAIL(EMBLA_UNSUPPORTED, "embla_attn_sparse_decode: the pool is not 16-bit");
    if (pool->n_kv_heads != ctx->cfg.n_kv_heads || view->layer < 0 || view->layer >= pool->n_layers)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_sparse_decode: pool/layer mismatch");
    if (view->batch <= 0 || view->batch > ctx->cfg.max_batch || !view->block_table_dev || !view->seq_lens_dev)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_sparse_decode: bad view (batch %d)", view->batch);
    const int max_len = view->max_seq_len > 0 ? view->max_seq_len : ctx->cfg.max_context;
    if (max_len > EMBLA_TOPK + EMBLA_RECENT && !idx_dev)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_sparse_decode: sequences past %d keys need the selected rows",
                   EMBLA_TOPK + EMBLA_RECENT);
    Attn16Params p = {};
    p.pool = pool->base;
    p.block_table = view->block_table_dev;
    p.table_stride = view->table_stride;
    p.idx = idx_dev;
    p.seq_lens = view->seq_lens_dev;
    p.q = q->q_dev;
    p.g1 = q->g1_dev;
    p.g2 = q->g2_dev;
    p.prenormed = q->prenormed;
    p.ng = q->ng;
    p.q_stride = q->q_stride;
    p.o = o_dev;
    p.o_stride = o_stride;
    p.page_bytes = pool->page_bytes;
    p.layer = view->layer;
    p.n_layers = pool->n_layers;
    return launch_attn16<A16_SPARSE>(ctx, p, view->batch, max_len < EMBLA_TOPK + EMBLA_RECENT ? max_len : EMBLA_TOPK + EMBLA_RECENT,
                                     static_cast<cudaStream_t>(stream));
}

// The full layers' ReLU² decode over a 16-bit pool (attn_full, attention.metal:148-220; the reference's EMBLA_KV8=0 build):
// every key of the sequence through the gathered-rows path, split into ranges as the sparse layers' attend. Reached
// through embla_attn_full_decode / embla_attn_full_step, which have checked their arguments.
namespace embla {
EmblaStatus attn16_full_decode(EmblaAttn* ctx, const EmblaKVPool* pool, const EmblaKVView* view, const EmblaQuery* q, void* o_dev,
                               int64_t o_stride, int max_len, cudaStream_t stream) {
    Attn16Params p = {};
    p.pool = pool->base;
    p.block_table = view->block_table_dev;
    p.table_stride = view->table_stride;
    p.idx = nullptr;
    p.seq_lens = view->seq_lens_dev;
    p.q = q->q_dev;
    p.g1 = q->g1_dev;
    p.g2 = q->g2_dev;
    p.prenormed = q->prenormed;
    p.ng = q->ng;
    p.q_stride = q->q_stride;
    p.o = o_dev;
    p.o_stride = o_stride;
    p.page_bytes = pool->page_bytes;
    p.layer = view->layer;
    p.n_layers = pool->n_layers;
    return launch_attn16<A16_FULL>(ctx, p, view->batch, max_len, stream);
}
}  // namespace embla

extern "C" EmblaStatus embla_sliding_write(EmblaAttn* ctx, const EmblaRing* ring, const int32_t* pos0_dev, int32_t batch,
                                           int32_t n_tokens, const void* k_dev, const void* v_dev, int64_t token_stride,
                                           int64_t seq_stride, int32_t prenormed, const void* kgain_dev, void* stream) {
    if (!ctx || !ring || !ring->k_dev || !ring->v_dev || !pos0_dev || !k_dev || !v_dev)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_sliding_write: null argument");
    EMBLA_CHECK_DEVICE("embla_sliding_write", ctx, static_cast<const EmblaKVPool*>(nullptr));
    if (batch <= 0 || n_tokens <= 0 || ring->ring <= 0 || (!prenormed && !kgain_dev))
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_sliding_write: batch %d, n_tokens %d, ring %d", batch, n_tokens, ring->ring);
    SlidingWriteParams p;
    p.k = k_dev;
    p.v = v_dev;
    p.kg = kgain_dev;
    p.ring_k = static_cast<uint8_t*>(ring->k_dev);
    p.ring_v = static_cast<uint8_t*>(ring->v_dev);
    p.pos0 = pos0_dev;
    p.token_stride = token_stride;
    p.seq_stride = seq_stride;
    p.ring_stride = ring->seq_stride;
    p.batch = batch;
    p.n_tokens = n_tokens;
    p.n_kv_heads = ctx->cfg.n_kv_heads;
    p.ring = ring->ring;
    p.prenormed = prenormed;
    fill_rope_freq(p.rope_freq);
    const long warps = long(batch) * n_tokens * p.n_kv_heads;
    const unsigned blocks = unsigned((warps + 3) / 4);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (ctx->cfg.act_dtype == EMBLA_BF16) sliding_write_kernel<EMBLA_BF16><<<blocks, 128, 0, s>>>(p);
    else sliding_write_kernel<EMBLA_F16><<<blocks, 128, 0, s>>>(p);
    EMBLA_CUDA_TRY(cudaGetLastError());
    return EMBLA_OK;
}

static EmblaStatus sliding_decode_impl(EmblaAttn* ctx, const EmblaRing* ring, const int32_t* seq_lens_dev, int32_t batch,
                                       const EmblaQuery* q, void* o_dev, int64_t o_stride, const void* k_new,
                                       const void* v_new, int64_t kv_stride, int32_t k_prenormed, const void* kgain,
                                       void* stream);

extern "C" EmblaStatus embla_attn_sliding_decode(EmblaAttn* ctx, const EmblaRing* ring, const int32_t* seq_lens_dev,
                                                 int32_t batch, const EmblaQuery* q, void* o_dev, int64_t o_stride,
                                                 void* stream) {
    return sliding_decode_impl(ctx, ring, seq_lens_dev, batch, q, o_dev, o_stride, nullptr, nullptr, 0, 1, nullptr, stream);
}

extern "C" EmblaStatus embla_attn_sliding_step(EmblaAttn* ctx, const EmblaRing* ring, const int32_t* seq_lens_dev,
                                               int32_t batch, const EmblaQuery* q, const void* k_dev, const void* v_dev,
                                               int64_t kv_stride, int32_t k_prenormed, const void* kgain_dev, void* o_dev,
                                               int64_t o_stride, void* stream) {
    if (!k_dev || !v_dev || (!k_prenormed && !kgain_dev)) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_sliding_step: null k, v or key gain");
    return sliding_decode_impl(ctx, ring, seq_lens_dev, batch, q, o_dev, o_stride, k_dev, v_dev, kv_stride, k_prenormed,
                               kgain_dev, stream);
}

static EmblaStatus sliding_decode_impl(EmblaAttn* ctx, const EmblaRing* ring, const int32_t* seq_lens_dev, int32_t batch,
                                       const EmblaQuery* q, void* o_dev, int64_t o_stride, const void* k_new,
                                       const void* v_new, int64_t kv_stride, int32_t k_prenormed, const void* kgain,
                                       void* stream) {
    if (!ctx || !ring || !ring->k_dev || !ring->v_dev || !seq_lens_dev || !o_dev)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_sliding_decode: null argument");
    EMBLA_CHECK_DEVICE("embla_attn_sliding_decode", ctx, static_cast<const EmblaKVPool*>(nullptr));
    if (EmblaStatus st = check_query("embla_attn_sliding_decode", q)) return st;
    // sliding layers norm q with ONE gain vector whatever ng says (attention.metal:47-48): it must be there
    if (!q->prenormed && !q->g1_dev)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_sliding_decode: q is not prenormed and g1_dev (the q gain) is null");
    if (batch <= 0 || batch > ctx->cfg.max_batch || ring->window <= 0 || ring->window > ring->ring)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_sliding_decode: batch %d, window %d, ring %d", batch, ring->window, ring->ring);
    // ring rows are fetched 16 bytes (or whole tiles) at a time
    if (reinterpret_cast<uintptr_t>(ring->k_dev) % 16 || reinterpret_cast<uintptr_t>(ring->v_dev) % 16 || ring->seq_stride % 8)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_sliding_decode: rings must start on 16 bytes, seq_stride %lld a multiple of 8",
                   (long long)ring->seq_stride);
    Attn16Params p = {};
    p.ring_k = static_cast<const uint8_t*>(ring->k_dev);
    p.ring_v = static_cast<const uint8_t*>(ring->v_dev);
    p.ring = ring->ring;
    p.window = ring->window;
    p.ring_stride = ring->seq_stride;
    p.seq_lens = seq_lens_dev;
    p.q = q->q_dev;
    p.g1 = q->g1_dev;
    p.g2 = q->g1_dev;
    p.prenormed = q->prenormed;
    p.ng = 1;
    p.q_stride = q->q_stride;
    p.o = o_dev;
    p.o_stride = o_stride;
    p.k_new = k_new;
    p.v_new = v_new;
    p.kgain = kgain;
    p.kv_stride = kv_stride;
    p.k_prenormed = k_prenormed;
    return launch_attn16<A16_SLIDING>(ctx, p, batch, ring->window, static_cast<cudaStream_t>(stream));
}
