// Key selection of the sparse layers: per (sequence, kv head), the 1024 highest-scoring keys among
// all but the 128 latest, then the 128 latest. Replaces select_keys
// (Sources/EmblaMetal/Kernels/attention.metal:655-744; dispatch Sources/EmblaMetal/Engine.swift:819-827).
//
// Integer work on the scores' order-preserving bit patterns, so the result is exact by construction:
// four 8-bit most-significant-digit-first histogram passes narrow down the 1024-th largest pattern,
// then a compaction in key order takes every key above it and the first equal ones. One CTA of 1024
// threads per (sequence, kv head); the patterns stay in registers after the one read of the scores.
// The output order is the reference's:
// [greater, ascending index][equal, ascending index][n .. n + 127].
#include <cooperative_groups.h>

#include "common.cuh"

namespace embla {

constexpr int SEL_T = 1024;
constexpr int SEL_WARPS = SEL_T / 32;

struct SelectParams {
    const float* scores;
    const int32_t* seq_lens;
    uint32_t* idx;
    int64_t scores_stride;   // floats between (sequence, kv head) rows
    int n_kv_heads;
};

__device__ __forceinline__ uint32_t order_bits(float f) {   // attention.metal:657-660
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// ITEMS: keys a lane holds in registers; warp w owns keys [w * 32 * ITEMS, (w + 1) * 32 * ITEMS), a
// round i takes the 32 consecutive keys w * 32 * ITEMS + 32 i + lane. The scores are read from global
// memory once, all loads in flight together; every pass after that runs on registers.
template <int ITEMS>
__global__ void __launch_bounds__(SEL_T) select_keys_kernel(const SelectParams p) {
    __shared__ uint32_t hist[SEL_WARPS][256];      // one histogram a warp: no contention across warps
    __shared__ uint32_t cum[256];
    __shared__ uint32_t sel[2];                    // digit, count above it

    const int kvh = blockIdx.x, b = blockIdx.y;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int S = p.seq_lens[b];
    if (S <= EMBLA_TOPK + EMBLA_RECENT) return;    // the reference does not select yet (Engine.swift:796)
    const int n = S - EMBLA_RECENT;
    const float* sc = p.scores + (size_t(b) * p.n_kv_heads + kvh) * p.scores_stride;
    uint32_t* out = p.idx + (size_t(b) * p.n_kv_heads + kvh) * (EMBLA_TOPK + EMBLA_RECENT);

    const int w0 = warp * 32 * ITEMS;
    uint32_t v[ITEMS];
#pragma unroll
    for (int i = 0; i < ITEMS; i++) {
        const int j = w0 + 32 * i + lane;
        v[i] = j < n ? order_bits(__ldg(sc + j)) : 0u;
    }
    for (int i = t; i < SEL_WARPS * 256; i += SEL_T) (&hist[0][0])[i] = 0;
    __syncthreads();

    uint32_t prefix = 0, mask = 0, k = EMBLA_TOPK;
    for (int shift = 24; shift >= 0; shift -= 8) {
#pragma unroll
        for (int i = 0; i < ITEMS; i++) {
            const bool in = w0 + 32 * i + lane < n && (v[i] & mask) == prefix;
            const uint32_t active = __ballot_sync(0xffffffffu, in);
            if (active == 0) continue;   // later passes: most rounds hold no candidate
            const uint32_t digit = (v[i] >> shift) & 255u;
            if (shift == 24) {
                // scores share a handful of leading digits: lanes with the same digit add once
                if (in) {
                    const uint32_t peers = __match_any_sync(active, digit);
                    if (lane == __ffs(peers) - 1) atomicAdd(&hist[warp][digit], uint32_t(__popc(peers)));
                }
            } else if (in) {
                atomicAdd(&hist[warp][digit], 1u);
            }
        }
        __syncthreads();
        if (t < 256) {
            uint32_t s = 0;
#pragma unroll 8
            for (int w = 0; w < SEL_WARPS; w++) {
                s += hist[w][t];
                hist[w][t] = 0;   // ready for the next pass
            }
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
    }
    // prefix is the TOPK-th largest pattern; every key above it, then the first k equal to it, in key order
    uint32_t gt = 0, eq = 0;
#pragma unroll
    for (int i = 0; i < ITEMS; i++) {
        const bool ok = w0 + 32 * i + lane < n;
        gt += __popc(__ballot_sync(0xffffffffu, ok && v[i] > prefix));
        eq += __popc(__ballot_sync(0xffffffffu, ok && v[i] == prefix));
    }
    __syncthreads();   // warp 0 has read cum[] of the last pass
    if (lane == 0) {
        cum[warp] = gt;
        cum[32 + warp] = eq;
    }
    __syncthreads();
    if (warp == 0) {   // exclusive scans of the 32 warps' counts
        uint32_t a = cum[lane], e = cum[32 + lane], ia = a, ie = e;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t ya = __shfl_up_sync(0xffffffffu, ia, o), ye = __shfl_up_sync(0xffffffffu, ie, o);
            if (lane >= o) {
                ia += ya;
                ie += ye;
            }
        }
        cum[64 + lane] = ia - a;
        cum[96 + lane] = ie - e;
        if (lane == 31) cum[128] = ia;
    }
    __syncthreads();
    uint32_t gpos = cum[64 + warp], epos = cum[96 + warp];
    const uint32_t ngt = cum[128], lt_mask = (1u << lane) - 1u;
#pragma unroll
    for (int i = 0; i < ITEMS; i++) {
        const int j = w0 + 32 * i + lane;
        const bool g = j < n && v[i] > prefix, e = j < n && v[i] == prefix;
        const uint32_t bg = __ballot_sync(0xffffffffu, g), be = __ballot_sync(0xffffffffu, e);
        if (g) out[gpos + __popc(bg & lt_mask)] = uint32_t(j);
        if (e) {
            const uint32_t at = epos + __popc(be & lt_mask);
            if (at < k) out[ngt + at] = uint32_t(j);
        }
        gpos += __popc(bg);
        epos += __popc(be);
    }
    for (int j = t; j < EMBLA_RECENT; j += SEL_T) out[EMBLA_TOPK + j] = uint32_t(n + j);
}

// The same selection by a thread-block cluster of CL CTAs per (sequence, kv head), for small batches where one CTA
// per pair would leave most SMs idle: CTA `rank` holds keys [rank * 1024 * 32 * ITEMS / 32 ...) — i.e. a contiguous
// 1024 * ITEMS keys — histograms are added across the cluster through distributed shared memory, every CTA
// derives the same digit, and the compaction offsets come from all CTAs' per-warp counts, so the output order
// (greater ascending, equal ascending, recent) is unchanged. Barriers are hardware cluster barriers, no spinning.
template <int ITEMS>
__global__ void __launch_bounds__(SEL_T) select_keys_cluster_kernel(const SelectParams p) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ uint32_t hist[SEL_WARPS][256];
    __shared__ uint32_t cum[2][256];               // this CTA's digit counts, double-buffered across passes
    __shared__ uint32_t wcnt[2][SEL_WARPS];        // this CTA's per-warp counts of greater / equal keys
    __shared__ uint32_t tot[256];
    __shared__ uint32_t sel[2];
    __shared__ uint32_t base[2][SEL_WARPS + 1];

    const int CL = int(cluster.num_blocks()), rank = int(cluster.block_rank());
    const int kvh = blockIdx.x / CL, b = blockIdx.y;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int S = p.seq_lens[b];
    const bool active = S > EMBLA_TOPK + EMBLA_RECENT;   // uniform over the cluster: every CTA keeps taking the barriers
    const int n = active ? S - EMBLA_RECENT : 0;
    const float* sc = p.scores + (size_t(b) * p.n_kv_heads + kvh) * p.scores_stride;
    uint32_t* out = p.idx + (size_t(b) * p.n_kv_heads + kvh) * (EMBLA_TOPK + EMBLA_RECENT);

    const int w0 = (rank * SEL_WARPS + warp) * 32 * ITEMS;
    uint32_t v[ITEMS];
#pragma unroll
    for (int i = 0; i < ITEMS; i++) {
        const int j = w0 + 32 * i + lane;
        v[i] = j < n ? order_bits(__ldg(sc + j)) : 0u;
    }
    for (int i = t; i < SEL_WARPS * 256; i += SEL_T) (&hist[0][0])[i] = 0;
    __syncthreads();

    uint32_t prefix = 0, mask = 0, k = EMBLA_TOPK;
    int pass = 0;
    for (int shift = 24; shift >= 0; shift -= 8, pass++) {
#pragma unroll
        for (int i = 0; i < ITEMS; i++) {
            const bool in = w0 + 32 * i + lane < n && (v[i] & mask) == prefix;
            const uint32_t act = __ballot_sync(0xffffffffu, in);
            if (act == 0) continue;
            const uint32_t digit = (v[i] >> shift) & 255u;
            if (shift == 24) {
                if (in) {
                    const uint32_t peers = __match_any_sync(act, digit);
                    if (lane == __ffs(peers) - 1) atomicAdd(&hist[warp][digit], uint32_t(__popc(peers)));
                }
            } else if (in) {
                atomicAdd(&hist[warp][digit], 1u);
            }
        }
        __syncthreads();
        if (t < 256) {
            uint32_t s = 0;
#pragma unroll 8
            for (int w = 0; w < SEL_WARPS; w++) {
                s += hist[w][t];
                hist[w][t] = 0;
            }
            cum[pass & 1][t] = s;
        }
        cluster.sync();
        if (t < 256) {
            uint32_t s = 0;
            for (int r = 0; r < CL; r++) s += cluster.map_shared_rank(&cum[pass & 1][0], r)[t];
            tot[t] = s;
        }
        __syncthreads();
        if (warp == 0) {
            uint32_t c[8], s = 0;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                c[i] = tot[255 - (lane * 8 + i)];
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
        if (active) {
            prefix |= sel[0] << shift;
            mask |= 255u << shift;
            k -= sel[1];
        }
    }
    uint32_t gt = 0, eq = 0;
#pragma unroll
    for (int i = 0; i < ITEMS; i++) {
        const bool ok = w0 + 32 * i + lane < n;
        gt += __popc(__ballot_sync(0xffffffffu, ok && v[i] > prefix));
        eq += __popc(__ballot_sync(0xffffffffu, ok && v[i] == prefix));
    }
    if (lane == 0) {
        wcnt[0][warp] = gt;
        wcnt[1][warp] = eq;
    }
    cluster.sync();
    // offsets of this CTA's warps: everything counted by lower ranks, then this CTA's lower warps
    if (warp < 2) {
        uint32_t before = 0, all = 0;
        for (int r = 0; r < CL; r++) {
            const uint32_t c = cluster.map_shared_rank(&wcnt[warp][0], r)[lane];
            uint32_t sum = c;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            if (r < rank) before += sum;
            all += sum;
        }
        const uint32_t mine = wcnt[warp][lane];
        uint32_t incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t y = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += y;
        }
        base[warp][lane] = before + incl - mine;
        if (lane == 0) base[warp][SEL_WARPS] = all;
    }
    __syncthreads();
    if (active) {
        uint32_t gpos = base[0][warp], epos = base[1][warp];
        const uint32_t ngt = base[0][SEL_WARPS], lt_mask = (1u << lane) - 1u;
#pragma unroll
        for (int i = 0; i < ITEMS; i++) {
            const int j = w0 + 32 * i + lane;
            const bool g = j < n && v[i] > prefix, e = j < n && v[i] == prefix;
            const uint32_t bg = __ballot_sync(0xffffffffu, g), be = __ballot_sync(0xffffffffu, e);
            if (g) out[gpos + __popc(bg & lt_mask)] = uint32_t(j);
            if (e) {
                const uint32_t at = epos + __popc(be & lt_mask);
                if (at < k) out[ngt + at] = uint32_t(j);
            }
            gpos += __popc(bg);
            epos += __popc(be);
        }
        if (rank == 0)
            for (int j = t; j < EMBLA_RECENT; j += SEL_T) out[EMBLA_TOPK + j] = uint32_t(n + j);
    }
    cluster.sync();   // no CTA leaves while another may still read its shared memory
}

template <int ITEMS>
static cudaError_t launch_select_cluster(const SelectParams& p, int batch, int cl, cudaStream_t s) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.n_kv_heads * cl, batch);
    cfg.blockDim = dim3(SEL_T);
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = cl;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, select_keys_cluster_kernel<ITEMS>, p);
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
    dim3 grid(p.n_kv_heads, batch);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int n_max = max_len - EMBLA_RECENT;   // keys a pair ranks: CL CTAs x 1024 threads x ITEMS
    if (n_max > 1024 * 32) EMBLA_FAIL(EMBLA_UNSUPPORTED, "embla_select_keys: %d keys (at most %d)", max_len, 1024 * 32 + EMBLA_RECENT);
    // small batches: a cluster of 2, 4 or 8 CTAs per (sequence, kv head), as many as keep the GPU busy
    int cl = 1;
    while (cl < 8 && 2 * cl * p.n_kv_heads * batch <= ctx->sm_count && n_max > 1024 * cl) cl *= 2;
    const int per_thread = (n_max + 1024 * cl - 1) / (1024 * cl);
    if (cl > 1) {
        cudaError_t e;
        if (per_thread <= 1) e = launch_select_cluster<1>(p, batch, cl, s);
        else if (per_thread <= 2) e = launch_select_cluster<2>(p, batch, cl, s);
        else if (per_thread <= 4) e = launch_select_cluster<4>(p, batch, cl, s);
        else if (per_thread <= 8) e = launch_select_cluster<8>(p, batch, cl, s);
        else e = launch_select_cluster<16>(p, batch, cl, s);
        EMBLA_CUDA_TRY(e);
    } else if (n_max <= 1024 * 4) select_keys_kernel<4><<<grid, SEL_T, 0, s>>>(p);
    else if (n_max <= 1024 * 8) select_keys_kernel<8><<<grid, SEL_T, 0, s>>>(p);
    else if (n_max <= 1024 * 16) select_keys_kernel<16><<<grid, SEL_T, 0, s>>>(p);
    else select_keys_kernel<32><<<grid, SEL_T, 0, s>>>(p);
    EMBLA_CUDA_TRY(cudaGetLastError());
    return EMBLA_OK;
}
