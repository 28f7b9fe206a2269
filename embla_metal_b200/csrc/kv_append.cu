// Quantised KV append: the reference's kv_append / kv_append_b with write_row8
// (Sources/EmblaMetal/Kernels/attention.metal:113-140, prefill.metal:184-212, common.metal:74-84),
// writing into the paged pool. One warp per (sequence, token, kv head, K|V); a lane holds dims
// lane + 32 i like the reference. Every fp32 operation is an explicit round-to-nearest intrinsic in
// the order the CPU oracle uses, so codes and scales are bit-exact. A 16-bit pool (sparse layers that
// keep their own keys) takes the rows as they are, rounded to the activation dtype.
#include "kv_row.cuh"

namespace embla {

struct AppendParams {
    uint8_t* pool;
    const int32_t* block_table;
    const int32_t* pos0;
    const void* k;
    const void* v;
    int64_t token_stride, seq_stride;
    size_t page_bytes;
    int table_stride, batch, n_tokens, layer, n_layers, n_kv_heads, scale_bytes, norm_k, kv16;
};

template <int DT>
__global__ void __launch_bounds__(128) kv_append_kernel(const AppendParams p) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const long warp = (long(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const long total = long(p.batch) * p.n_tokens * p.n_kv_heads * 2;
    if (warp >= total) return;
    const int is_v = int(warp & 1);
    const int h = int((warp >> 1) % p.n_kv_heads);
    const long bt = (warp >> 1) / p.n_kv_heads;
    const int t = int(bt % p.n_tokens), b = int(bt / p.n_tokens);
    const void* src = is_v ? p.v : p.k;
    const size_t off = size_t(b) * p.seq_stride + size_t(t) * p.token_stride + size_t(h) * HD;

    float x[4];
    kv_row_load<DT>(src, off, !is_v && p.norm_k, lane, x);
    const int pos = p.pos0[b] + t;
    const int block = p.block_table[size_t(b) * p.table_stride + pos / BLK];
    const int row = pos % BLK;
    uint8_t* page = p.pool + ((size_t(block) * p.n_layers + p.layer) * p.n_kv_heads + h) * p.page_bytes;
    if (p.kv16) {   // 16-bit pages: K rows [128][128], then V rows, in the activation dtype
        uint8_t* dst = page + (is_v ? BLK * HD * 2 : 0);
#pragma unroll
        for (int i = 0; i < 4; i++) Act<DT>::store(dst, size_t(row) * HD + lane + 32 * i, x[i]);
        return;
    }
    int code[4];
    float scale;
    kv_row_quantise<DT>(x, code, scale);
    int8_t* codes = reinterpret_cast<int8_t*>(page) + (is_v ? CODE_BYTES : 0) + row * HD;
#pragma unroll
    for (int i = 0; i < 4; i++) codes[lane + 32 * i] = int8_t(code[i]);
    if (lane == 0) {
        uint8_t* sc = page + 2 * CODE_BYTES + (is_v ? BLK * p.scale_bytes : 0);
        if (p.scale_bytes == 4) reinterpret_cast<float*>(sc)[row] = scale;
        else reinterpret_cast<__half*>(sc)[row] = __float2half_rn(scale);
    }
}

}  // namespace embla

using namespace embla;

extern "C" EmblaStatus embla_kv_append(EmblaAttn* ctx, EmblaKVPool* pool, const EmblaKVView* view,
                                       const int32_t* pos0_dev, int32_t n_tokens,
                                       const void* k_dev, const void* v_dev, int64_t token_stride, int64_t seq_stride,
                                       int32_t norm_k, void* stream) {
    if (!ctx || !pool || !view || !pos0_dev || !k_dev || !v_dev) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_kv_append: null argument");
    EMBLA_CHECK_DEVICE("embla_kv_append", ctx, pool);
    if (view->layer < 0 || view->layer >= pool->n_layers)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_kv_append: layer %d outside the pool's %d", view->layer, pool->n_layers);
    if (view->batch <= 0 || n_tokens <= 0 || !view->block_table_dev)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_kv_append: batch %d, n_tokens %d", view->batch, n_tokens);
    if (pool->n_kv_heads != ctx->cfg.n_kv_heads)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_kv_append: pool has %d kv heads, context %d", pool->n_kv_heads, ctx->cfg.n_kv_heads);
    AppendParams p;
    p.pool = pool->base;
    p.block_table = view->block_table_dev;
    p.pos0 = pos0_dev;
    p.k = k_dev;
    p.v = v_dev;
    p.token_stride = token_stride;
    p.seq_stride = seq_stride;
    p.page_bytes = pool->page_bytes;
    p.table_stride = view->table_stride;
    p.batch = view->batch;
    p.n_tokens = n_tokens;
    p.layer = view->layer;
    p.n_layers = pool->n_layers;
    p.n_kv_heads = pool->n_kv_heads;
    p.scale_bytes = pool->scale_bytes;
    p.norm_k = norm_k;
    p.kv16 = pool->kv_dtype == EMBLA_KV_16BIT;
    const long warps = long(p.batch) * n_tokens * p.n_kv_heads * 2;
    const unsigned blocks = unsigned((warps + 3) / 4);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (ctx->cfg.act_dtype == EMBLA_BF16) EMBLA_CUDA_TRY(launch_kernel(ctx->pdl, kv_append_kernel<EMBLA_BF16>, dim3(blocks), dim3(128), 0, s, p));
    else EMBLA_CUDA_TRY(launch_kernel(ctx->pdl, kv_append_kernel<EMBLA_F16>, dim3(blocks), dim3(128), 0, s, p));
    EMBLA_CUDA_TRY(cudaGetLastError());
    return EMBLA_OK;
}
