// Key selection of the sparse layers: per (sequence, kv head), the 1024 highest-scoring keys among
// all but the 128 latest, then the 128 latest. Replaces select_keys
// (Sources/EmblaMetal/Kernels/attention.metal:655-744; dispatch Sources/EmblaMetal/Engine.swift:819-827).
//
// Integer work on the scores' order-preserving bit patterns, so the result is exact by construction:
// four 8-bit most-significant-digit-first histogram passes narrow down the 1024-th largest pattern,
// then a compaction in key order takes every key above it and the first equal ones. One CTA of 1024
// threads per (sequence, kv head); the patterns are kept in shared memory after the first read when
// they fit, so HBM/L2 is read once. The output order is the reference's:
// [greater, ascending index][equal, ascending index][n .. n + 127].
#include "common.cuh"

namespace embla {

constexpr int SEL_T = 1024;
constexpr int SEL_WARPS = SEL_T / 32;

struct SelectParams {
    const float* scores;
    const int32_t* seq_lens;
    uint32_t* idx;
    int64_t scores_stride;   // floats between (sequence, kv head) rows
    int n_kv_heads, cache_cap;
};

__device__ __forceinline__ uint32_t order_bits(float f) {   // attention.metal:657-660
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Exclusive prefix sum of one value per thread over the CTA, and the total.
__device__ __forceinline__ uint32_t block_scan_excl(uint32_t v, uint32_t* buf, int lane, int warp, uint32_t& total) {
    uint32_t incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t y = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += y;
    }
    if (lane == 31) buf[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        const uint32_t s = buf[lane];
        uint32_t p = s;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t y = __shfl_up_sync(0xffffffffu, p, o);
            if (lane >= o) p += y;
        }
        buf[lane] = p - s;
        if (lane == 31) buf[32] = p;
    }
    __syncthreads();
    const uint32_t r = buf[warp] + incl - v;
    total = buf[32];
    __syncthreads();
    return r;
}

template <bool CACHED>
__global__ void __launch_bounds__(SEL_T) select_keys_kernel(const SelectParams p) {
    extern __shared__ uint32_t cache[];            // CACHED: the order bits of all n scores
    __shared__ uint32_t hist[SEL_WARPS][256];      // one histogram a warp: no contention across warps
    __shared__ uint32_t cum[256];
    __shared__ uint32_t buf[33];
    __shared__ uint32_t sel[2];                    // digit, count above it

    const int kvh = blockIdx.x, b = blockIdx.y;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int S = p.seq_lens[b];
    if (S <= EMBLA_TOPK + EMBLA_RECENT) return;    // the reference does not select yet (Engine.swift:796)
    const int n = S - EMBLA_RECENT;
    const float* sc = p.scores + (size_t(b) * p.n_kv_heads + kvh) * p.scores_stride;
    uint32_t* out = p.idx + (size_t(b) * p.n_kv_heads + kvh) * (EMBLA_TOPK + EMBLA_RECENT);

    if (CACHED) {
        for (int j = t; j < n; j += SEL_T) cache[j] = order_bits(sc[j]);
        __syncthreads();
    }
    auto bits_at = [&](int j) -> uint32_t { return CACHED ? cache[j] : order_bits(sc[j]); };

    uint32_t prefix = 0, mask = 0, k = EMBLA_TOPK;
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int i = t; i < SEL_WARPS * 256; i += SEL_T) (&hist[0][0])[i] = 0;
        __syncthreads();
        for (int j = t; j < n; j += SEL_T) {
            const uint32_t v = bits_at(j);
            if ((v & mask) == prefix) atomicAdd(&hist[warp][(v >> shift) & 255u], 1u);
        }
        __syncthreads();
        if (t < 256) {
            uint32_t s = 0;
#pragma unroll 8
            for (int w = 0; w < SEL_WARPS; w++) s += hist[w][t];
            cum[t] = s;
        }
        __syncthreads();
        // counts above each digit, from the top: the digit whose bucket holds the k-th largest
        if (warp == 0) {
            uint32_t c[8], s = 0;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                c[i] = cum[255 - (lane * 8 + i)];
                s += c[i];
            }
            uint32_t incl = s;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t y = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += y;
            }
            uint32_t above = incl - s;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                if (above < k && above + c[i] >= k) {
                    sel[0] = 255 - (lane * 8 + i);
                    sel[1] = above;
                }
                above += c[i];
            }
        }
        __syncthreads();
        prefix |= sel[0] << shift;
        mask |= 255u << shift;
        k -= sel[1];
        __syncthreads();
    }
    // prefix is the TOPK-th largest pattern; every key above it, then the first k equal to it, in key order
    const int per = (n + SEL_T - 1) / SEL_T, j0 = t * per, j1 = min(n, j0 + per);
    uint32_t gt = 0, eq = 0;
    for (int j = j0; j < j1; j++) {
        const uint32_t v = bits_at(j);
        gt += v > prefix;
        eq += v == prefix;
    }
    uint32_t ngt, neq;
    uint32_t gpos = block_scan_excl(gt, buf, lane, warp, ngt);
    uint32_t epos = block_scan_excl(eq, buf, lane, warp, neq);
    for (int j = j0; j < j1; j++) {
        const uint32_t v = bits_at(j);
        if (v > prefix) out[gpos++] = uint32_t(j);
        else if (v == prefix) {
            if (epos < k) out[ngt + epos] = uint32_t(j);
            epos++;
        }
    }
    for (int j = t; j < EMBLA_RECENT; j += SEL_T) out[EMBLA_TOPK + j] = uint32_t(n + j);
}

}  // namespace embla

using namespace embla;

extern "C" EmblaStatus embla_select_keys(EmblaAttn* ctx, const float* scores_dev, int64_t scores_stride,
                                         const int32_t* seq_lens_dev, int32_t batch, int32_t max_seq_len,
                                         uint32_t* idx_dev, void* stream) {
    if (!ctx || !scores_dev || !seq_lens_dev || !idx_dev) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_select_keys: null argument");
    if (batch <= 0) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_select_keys: batch %d", batch);
    const int max_len = max_seq_len > 0 ? max_seq_len : ctx->cfg.max_context;
    if (scores_stride < max_len) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_select_keys: scores_stride %lld under max_seq_len %d",
                                            (long long)scores_stride, max_len);
    SelectParams p;
    p.scores = scores_dev;
    p.seq_lens = seq_lens_dev;
    p.idx = idx_dev;
    p.scores_stride = scores_stride;
    p.n_kv_heads = ctx->cfg.n_kv_heads;
    const size_t cache_bytes = size_t(max_len) * 4;
    constexpr size_t kMaxCache = 180 * 1024;
    dim3 grid(p.n_kv_heads, batch);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (cache_bytes <= kMaxCache) {
        static bool configured[64] = {};
        if (!configured[ctx->device & 63]) {
            EMBLA_CUDA_TRY(cudaFuncSetAttribute(select_keys_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                int(kMaxCache)));
            configured[ctx->device & 63] = true;
        }
        select_keys_kernel<true><<<grid, SEL_T, cache_bytes, s>>>(p);
    } else {
        select_keys_kernel<false><<<grid, SEL_T, 0, s>>>(p);
    }
    EMBLA_CUDA_TRY(cudaGetLastError());
    return EMBLA_OK;
}
