// Context, KV pool and block copies of the embla CUDA attention library.
#include <cstdlib>
#include <cstring>
#include <new>

#include "common.cuh"

namespace embla {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

TensorMapEncodeTiledFn tensor_map_encoder() {
    static TensorMapEncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<TensorMapEncodeTiledFn>(p);
    }
    return fn;
}

}  // namespace embla

using namespace embla;

extern "C" {

const char* embla_version(void) { return "embla-cuda-attn 0.1 (sm_100a)"; }
const char* embla_last_error(void) { return g_error; }

EmblaStatus embla_attn_create(const EmblaAttnConfig* cfg, EmblaAttn** out) {
    if (!cfg || !out) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_create: null argument");
    *out = nullptr;
    if (cfg->n_kv_heads <= 0 || cfg->n_q_heads <= 0 || cfg->n_q_heads % cfg->n_kv_heads != 0)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_create: n_q_heads %d must be a positive multiple of n_kv_heads %d",
                   cfg->n_q_heads, cfg->n_kv_heads);
    const int G = cfg->n_q_heads / cfg->n_kv_heads;
    if (G > 8) EMBLA_FAIL(EMBLA_UNSUPPORTED, "embla_attn_create: %d query heads per kv head (at most 8)", G);
    if (cfg->act_dtype != EMBLA_BF16 && cfg->act_dtype != EMBLA_F16)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_create: act_dtype %d", cfg->act_dtype);
    if (cfg->max_batch <= 0 || cfg->max_context <= 0)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_create: max_batch %d, max_context %d", cfg->max_batch, cfg->max_context);

    EmblaAttn* ctx = new (std::nothrow) EmblaAttn();
    if (!ctx) EMBLA_FAIL(EMBLA_OOM, "embla_attn_create: host allocation failed");
    ctx->cfg = *cfg;
    ctx->partials = nullptr;
    ctx->counters = nullptr;
    ctx->err_dev = nullptr;
    ctx->prefill_scratch = nullptr;
    ctx->prefill_scratch_bytes = 0;
    ctx->prefill_counters = 0;
    ctx->pdl = 0;
    ctx->early = 0;
    ctx->wait_cycles = WAIT_CYCLES;
    ctx->stall_at = -1;
    {
        const char* e = getenv("EMBLA_L2_PAGES");
        ctx->l2_pages = e ? atoi(e) : 8;
    }
    ctx->trace_dev = nullptr;
    ctx->trace_entry = nullptr;
    ctx->trace_cap = ctx->trace_next = ctx->trace_on = 0;
    ctx->trace_tag = -1;
    ctx->ring_maps_used = ctx->ring_maps_next = 0;
    cudaError_t e = cudaGetDevice(&ctx->device);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&ctx->sm_count, cudaDevAttrMultiProcessorCount, ctx->device);
    if (e != cudaSuccess) {
        delete ctx;
        EMBLA_FAIL(EMBLA_CUDA, "embla_attn_create: no usable CUDA device: %s", cudaGetErrorString(e));
    }
    // Split-K scratch: a (sequence, kv head) pair is cut into key ranges, each
    // leaving G rows of 128 sums + 2 scalars (sum of weights, or running max and sum for softmax).
    // Slots: enough key ranges to fill the GPU several times over at any batch up to max_batch.
    const long pairs = long(cfg->max_batch) * cfg->n_kv_heads;
    // (The softmax kernels cut a pair's rows into 128-row chunks: 9 for 1152 selected rows, window / 128
    // for a sliding layer; 16 chunks a pair covers windows up to 2048.)
    ctx->partial_slots = int(8L * ctx->sm_count + 16 * pairs);
    ctx->partial_floats = size_t(ctx->partial_slots) * G * (HD + 4);
    e = cudaMalloc(&ctx->partials, ctx->partial_floats * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&ctx->counters, size_t(pairs) * sizeof(int));
    if (e == cudaSuccess) e = cudaMalloc(&ctx->err_dev, sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(ctx->counters, 0, size_t(pairs) * sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(ctx->err_dev, 0, sizeof(int));
    if (e != cudaSuccess) {
        embla_attn_destroy(ctx);
        set_error("embla_attn_create: scratch allocation failed: %s", cudaGetErrorString(e));
        return e == cudaErrorMemoryAllocation ? EMBLA_OOM : EMBLA_CUDA;
    }
    *out = ctx;
    return EMBLA_OK;
}

void embla_attn_destroy(EmblaAttn* ctx) {
    if (!ctx) return;
    cudaFree(ctx->partials);
    cudaFree(ctx->counters);
    cudaFree(ctx->err_dev);
    cudaFree(ctx->prefill_scratch);
    cudaFree(ctx->trace_dev);
    delete[] ctx->trace_entry;
    delete ctx;
}

EmblaStatus embla_attn_set_wait_limit(EmblaAttn* ctx, int64_t cycles) {
    if (!ctx || cycles <= 0) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_set_wait_limit: null context or limit %lld", (long long)cycles);
    ctx->wait_cycles = cycles;
    return EMBLA_OK;
}

EmblaStatus embla_attn_inject_stall(EmblaAttn* ctx, int32_t item) {
    if (!ctx) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_inject_stall: null context");
    ctx->stall_at = item < 0 ? -1 : item;
    return EMBLA_OK;
}

EmblaStatus embla_attn_trace_begin(EmblaAttn* ctx, int32_t max_launches, void* stream) {
    if (!ctx || max_launches <= 0) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_trace_begin: null context or %d launches", max_launches);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (max_launches > ctx->trace_cap) {
        EMBLA_CUDA_TRY(cudaStreamSynchronize(s));
        cudaFree(ctx->trace_dev);
        delete[] ctx->trace_entry;
        ctx->trace_dev = nullptr;
        ctx->trace_entry = nullptr;
        ctx->trace_cap = 0;
        EMBLA_CUDA_TRY(cudaMalloc(&ctx->trace_dev, size_t(max_launches) * TRACE_SLOTS * sizeof(unsigned long long)));
        ctx->trace_entry = new (std::nothrow) int[max_launches];
        if (!ctx->trace_entry) EMBLA_FAIL(EMBLA_OOM, "embla_attn_trace_begin: host allocation failed");
        ctx->trace_cap = max_launches;
    }
    EMBLA_CUDA_TRY(cudaMemsetAsync(ctx->trace_dev, 0xff, size_t(ctx->trace_cap) * TRACE_SLOTS * sizeof(unsigned long long), s));
    ctx->trace_next = 0;
    ctx->trace_on = 1;
    return EMBLA_OK;
}

EmblaStatus embla_attn_trace_end(EmblaAttn* ctx, void* stream, uint64_t* stamps, int32_t* entries, int32_t cap, int32_t* n_out) {
    if (!ctx || !stamps || !entries || !n_out) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_trace_end: null argument");
    ctx->trace_on = 0;
    const int n = ctx->trace_next < cap ? ctx->trace_next : cap;
    *n_out = n;
    if (n == 0) return EMBLA_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    EMBLA_CUDA_TRY(cudaMemcpyAsync(stamps, ctx->trace_dev, size_t(n) * TRACE_SLOTS * sizeof(uint64_t), cudaMemcpyDeviceToHost, s));
    EMBLA_CUDA_TRY(cudaStreamSynchronize(s));
    for (int i = 0; i < n; i++) {
        entries[i] = ctx->trace_entry[i];
        // the "last CTA" slots (2, 3, 6, 7) are kept as complements on the device; a slot no CTA stamped reads 0
        for (int k = 0; k < TRACE_SLOTS; k++) {
            uint64_t& v = stamps[TRACE_SLOTS * i + k];
            if ((k & 2) != 0) v = ~v;
            else if (v == ~uint64_t(0)) v = 0;
        }
    }
    return EMBLA_OK;
}

EmblaStatus embla_attn_check(EmblaAttn* ctx, void* stream) {
    if (!ctx) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_check: null context");
    int err = 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    EMBLA_CUDA_TRY(cudaMemcpyAsync(&err, ctx->err_dev, sizeof(int), cudaMemcpyDeviceToHost, s));
    EMBLA_CUDA_TRY(cudaStreamSynchronize(s));
    if (err != 0) {
        EMBLA_CUDA_TRY(cudaMemsetAsync(ctx->err_dev, 0, sizeof(int), s));
        EMBLA_CUDA_TRY(cudaStreamSynchronize(s));
        EMBLA_FAIL(EMBLA_TIMEOUT, "a kernel gave up a bounded wait (code %d)", err);
    }
    return EMBLA_OK;
}

EmblaStatus embla_kv_pool_create(int32_t n_layers, int32_t n_kv_heads, int32_t kv_dtype, int32_t scale_dtype,
                                 int32_t num_blocks, EmblaKVPool** out) {
    if (!out) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_kv_pool_create: null output");
    *out = nullptr;
    if (n_layers <= 0 || n_kv_heads <= 0 || num_blocks <= 0)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_kv_pool_create: n_layers %d, n_kv_heads %d, num_blocks %d", n_layers, n_kv_heads,
                   num_blocks);
    if (kv_dtype != EMBLA_KV_INT8 && kv_dtype != EMBLA_KV_16BIT)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_kv_pool_create: kv_dtype %d", kv_dtype);
    if (scale_dtype != EMBLA_SCALE_F32 && scale_dtype != EMBLA_SCALE_F16)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_kv_pool_create: scale_dtype %d", scale_dtype);
    EmblaKVPool* p = new (std::nothrow) EmblaKVPool();
    if (!p) EMBLA_FAIL(EMBLA_OOM, "embla_kv_pool_create: host allocation failed");
    p->n_layers = n_layers;
    p->n_kv_heads = n_kv_heads;
    p->kv_dtype = kv_dtype;
    p->scale_dtype = scale_dtype;
    p->num_blocks = num_blocks;
    p->scale_bytes = scale_dtype == EMBLA_SCALE_F32 ? 4 : 2;
    p->page_bytes = kv_dtype == EMBLA_KV_INT8 ? size_t(2 * CODE_BYTES + 2 * BLK * p->scale_bytes) : size_t(2 * BLK * HD * 2);
    // tensor-map rows: 128 bytes for int8 pages, 256 bytes (one key) for 16-bit pages
    const int row_bytes = kv_dtype == EMBLA_KV_INT8 ? 128 : 256;
    p->rows_per_page = int(p->page_bytes / row_bytes);
    p->block_bytes = p->page_bytes * n_layers * n_kv_heads;
    p->total_bytes = p->block_bytes * num_blocks;
    p->base = nullptr;
    cudaError_t e = cudaGetDevice(&p->device);
    if (e == cudaSuccess) e = cudaMalloc(&p->base, p->total_bytes);
    if (e == cudaSuccess) e = cudaMemset(p->base, 0, p->total_bytes);
    if (e != cudaSuccess) {
        const size_t want = p->total_bytes;
        cudaFree(p->base);
        delete p;
        set_error("embla_kv_pool_create: %zu bytes: %s", want, cudaGetErrorString(e));
        return e == cudaErrorMemoryAllocation ? EMBLA_OOM : EMBLA_CUDA;
    }
    // The whole pool as rows of 128 bytes; one box = the 256 code rows (K then V) of an int8 page,
    // or half of a 16-bit page side. 128-byte swizzle: 16-byte chunk c of row r lands at c ^ (r % 8).
    TensorMapEncodeTiledFn enc = tensor_map_encoder();
    if (!enc) {
        cudaFree(p->base);
        delete p;
        EMBLA_FAIL(EMBLA_CUDA, "embla_kv_pool_create: cuTensorMapEncodeTiled is not available from this driver");
    }
    // (16-bit pages: rows of 256 bytes seen through 128-byte-wide boxes of 128 keys, so that a key's
    // dims 0-63 and 64-127 land in two tiles, each [128 keys][128 B] under the same swizzle.)
    const cuuint64_t dims[2] = {cuuint64_t(row_bytes), cuuint64_t(p->total_bytes / row_bytes)};
    const cuuint64_t strides[1] = {cuuint64_t(row_bytes)};
    const cuuint32_t box[2] = {128, kv_dtype == EMBLA_KV_INT8 ? 256u : 128u};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(&p->tmap_codes, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, p->base, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_SUCCESS) {
        const cuuint32_t box_half[2] = {128, 128};
        r = enc(&p->tmap_half, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, p->base, dims, strides, box_half, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if (r != CUDA_SUCCESS) {
        cudaFree(p->base);
        delete p;
        EMBLA_FAIL(EMBLA_CUDA, "embla_kv_pool_create: cuTensorMapEncodeTiled failed (%d)", int(r));
    }
    *out = p;
    return EMBLA_OK;
}

void embla_kv_pool_destroy(EmblaKVPool* pool) {
    if (!pool) return;
    cudaFree(pool->base);
    delete pool;
}

size_t embla_kv_block_bytes(const EmblaKVPool* pool) { return pool ? pool->block_bytes : 0; }
size_t embla_kv_page_bytes(const EmblaKVPool* pool) { return pool ? pool->page_bytes : 0; }
void* embla_kv_pool_base(const EmblaKVPool* pool) { return pool ? pool->base : nullptr; }

EmblaStatus embla_kv_block_export(const EmblaKVPool* pool, int32_t block, void* dst, void* stream) {
    if (!pool || !dst) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_kv_block_export: null argument");
    if (block < 0 || block >= pool->num_blocks)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_kv_block_export: block %d outside 0..%d", block, pool->num_blocks - 1);
    EMBLA_CUDA_TRY(cudaMemcpyAsync(dst, pool->base + size_t(block) * pool->block_bytes, pool->block_bytes,
                                   cudaMemcpyDefault, static_cast<cudaStream_t>(stream)));
    return EMBLA_OK;
}

EmblaStatus embla_kv_block_import(EmblaKVPool* pool, int32_t block, const void* src, void* stream) {
    if (!pool || !src) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_kv_block_import: null argument");
    if (block < 0 || block >= pool->num_blocks)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_kv_block_import: block %d outside 0..%d", block, pool->num_blocks - 1);
    EMBLA_CUDA_TRY(cudaMemcpyAsync(pool->base + size_t(block) * pool->block_bytes, src, pool->block_bytes,
                                   cudaMemcpyDefault, static_cast<cudaStream_t>(stream)));
    return EMBLA_OK;
}

}  // extern "C"
