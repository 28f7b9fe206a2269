// Key selection of the sparse layers: per (sequence, kv head), the 1024 highest-scoring keys among
// all but the 128 latest, then the 128 latest. Replaces select_keys
// (Sources/EmblaMetal/Kernels/attention.metal:655-744; dispatch Sources/EmblaMetal/Engine.swift:819-827).
//
// Integer work on the scores' order-preserving bit patterns, so the result is exact by construction:
// three most-significant-digit-first histogram passes (11, 11 and 10 bits) narrow down the 1024-th
// largest pattern, then a compaction in key order takes every key above it and the first equal ones.
// A cluster of 1, 2, 4 or 8 CTAs of 1024 threads per (sequence, kv head) - more CTAs the fewer pairs
// there are, so that small batches still fill the SMs; the patterns stay in registers after the one
// read of the scores; histograms are read across the cluster through distributed shared memory, the
// warps' counts for the ordered writes are written into every CTA of the cluster; barriers are
// hardware cluster barriers (no spinning). The output order is the reference's:
// [greater, ascending index][equal, ascending index][n .. n + 127].
#include <cooperative_groups.h>

#include "common.cuh"

namespace embla {

constexpr int SEL_T = 1024;
constexpr int SEL_WARPS = SEL_T / 32;
constexpr int SEL_BINS = 2048;

struct SelectParams {
    const float* scores;
    const int32_t* seq_lens;
    uint32_t* idx;
    int64_t scores_stride;   // floats between (sequence, kv head) rows
    int n_kv_heads;
    KernelCtl ctl;
};

__device__ __forceinline__ uint32_t order_bits(float f) {   // attention.metal:657-660
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ uint32_t warp_incl_scan(uint32_t x, int lane) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
    }
    return x;
}

// ITEMS: keys a lane holds in registers. CTA `rank` of the cluster owns 1024 * ITEMS contiguous keys, its warp w
// the keys [w0, w0 + 32 * ITEMS), and round i takes the 32 consecutive keys w0 + 32 i + lane. The scores are read
// from global memory once, all loads in flight together; every pass after that runs on registers.
// SINGLE: one CTA per pair (launched without a cluster) - block barriers and plain shared-memory loads take the place of
// the cluster barriers and of the loads through the cluster's shared-memory window.
template <int ITEMS, bool BULK, bool SINGLE>
__global__ void __launch_bounds__(SEL_T) select_keys_kernel(const SelectParams p) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ __align__(16) uint32_t hist[2][SEL_BINS];   // this CTA's digit counts, double-buffered across passes
    __shared__ uint32_t wsum[SEL_WARPS];
    __shared__ uint32_t sel[2];                            // digit, count above it
    __shared__ uint32_t wall[2][8][SEL_WARPS];             // per-warp counts of greater / equal keys of every CTA of the cluster
    __shared__ uint32_t base[2][SEL_WARPS + 1];

    const int CL = SINGLE ? 1 : int(cluster.num_blocks()), rank = SINGLE ? 0 : int(cluster.block_rank());
    const int kvh = blockIdx.x / CL, b = blockIdx.y;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    trace_first(p.ctl.trace, 0);
    const int S = p.seq_lens[b];   // (read ahead of the wait: nothing on the GPU writes the sequence lengths)
    pdl_wait();
    pdl_launch_dependents();
    trace_first(p.ctl.trace, 1);
    // the reference does not select yet at or below 1152 keys (Engine.swift:796); the whole cluster of a pair leaves
    if (S <= EMBLA_TOPK + EMBLA_RECENT) return;
    const int n = S - EMBLA_RECENT;
    const float* sc = p.scores + (size_t(b) * p.n_kv_heads + kvh) * p.scores_stride;
    uint32_t* out = p.idx + (size_t(b) * p.n_kv_heads + kvh) * (EMBLA_TOPK + EMBLA_RECENT);

    for (int i = t; i < 2 * SEL_BINS; i += SEL_T) (&hist[0][0])[i] = 0;
    const int w0 = (rank * SEL_WARPS + warp) * 32 * ITEMS;
    const int lim = n - w0 - lane;                 // key of round i exists while 32 i < lim
    uint32_t v[ITEMS];
    if (BULK) {
        // The CTA's scores come as bulk copies into shared memory (a lane's own 4-byte loads keep too few bytes in
        // flight per SM), then each lane takes its keys from there.
        extern __shared__ __align__(16) uint8_t staged_raw[];
        __shared__ uint64_t bar;
        float* staged = reinterpret_cast<float*>(staged_raw);
        const int cta0 = rank * SEL_T * ITEMS;
        const int cnt = min(max(n - cta0, 0), SEL_T * ITEMS);
        const uint32_t bytes = uint32_t((cnt + 3) & ~3) * 4u;   // whole 16-byte units: at most 3 scores past n, inside the row
        if (t == 0) {
            mbar_init(&bar, 1);
            fence_barrier_init();
            if (bytes) {
                mbar_expect_tx(&bar, bytes);
                for (uint32_t off = 0; off < bytes; off += 16384u)
                    bulk_load_1d(staged_raw + off, reinterpret_cast<const uint8_t*>(sc + cta0) + off, min(16384u, bytes - off), &bar);
            }
        }
        __syncthreads();
        if (bytes && !mbar_wait_bounded(p.ctl.wait_cycles, &bar, 0) && lane == 0) atomicExch(p.ctl.err, ERR_WAIT_FULL);
#pragma unroll
        for (int i = 0; i < ITEMS; i++) v[i] = 32 * i < lim ? order_bits(staged[warp * 32 * ITEMS + 32 * i + lane]) : 0u;
    } else {
        // every load issued before the first use (addresses clamped, not predicated: one batch in flight)
        const float* src = sc + (lim > 0 ? w0 + lane : 0);
        float raw[ITEMS];
#pragma unroll
        for (int i = 0; i < ITEMS; i++) raw[i] = __ldg(src + (32 * i < lim ? 32 * i : 0));
#pragma unroll
        for (int i = 0; i < ITEMS; i++) v[i] = 32 * i < lim ? order_bits(raw[i]) : 0u;
        __syncthreads();
    }
    const uint32_t wall_here = smem_u32(&wall[0][0][0]);

    uint32_t prefix = 0, mask = 0, k = EMBLA_TOPK;
#pragma unroll
    for (int pass = 0; pass < 3; pass++) {
        const int shift = pass == 0 ? 21 : pass == 1 ? 10 : 0;
        const int nb = pass == 2 ? 1024 : 2048;
        uint32_t* h = hist[pass & 1];
#pragma unroll
        for (int i = 0; i < ITEMS; i++) {
            const bool in = 32 * i < lim && (v[i] & mask) == prefix;
            const uint32_t act = __ballot_sync(0xffffffffu, in);
            if (act == 0) continue;   // later passes: most rounds hold no candidate
            const uint32_t digit = (v[i] >> shift) & uint32_t(nb - 1);
            if (act == 0xffffffffu) {
                // one digit for the whole round (constant or saturated scores): one add, not 32 colliding ones
                const uint32_t lo = __reduce_min_sync(0xffffffffu, digit), hi = __reduce_max_sync(0xffffffffu, digit);
                if (lo == hi) {
                    if (lane == 0) atomicAdd(&h[digit], 32u);
                    continue;
                }
            }
            if (in) atomicAdd(&h[digit], 1u);
        }
        if (pass == 1) trace_first(p.ctl.trace, 4);
        if (SINGLE) {
            __syncthreads();
        } else {
            cluster_arrive();
            cluster_wait();
        }
        if (pass == 1) trace_first(p.ctl.trace, 5);
        // counts above each digit, from the top, over the cluster: the digit whose bucket holds the k-th largest.
        // Thread t < nb / 4 takes digits nb - 1 - 4t .. nb - 4 - 4t, read as ONE 16-byte load a CTA, four CTAs' loads in
        // flight together (loads from another CTA's shared memory are bound by their number and their latency: read as
        // two 4-byte loads a digit pair they took 2.8 of a pass's 3.2 microseconds; adding the counts into every CTA's
        // array with remote atomics instead took longer still).
        uint32_t c[4] = {0, 0, 0, 0};   // c[j]: digit nb - 1 - 4t - j
        if (4 * t < nb) {
            const int word = nb - 4 - 4 * t;
            if (SINGLE) {
                const uint4 q4 = *reinterpret_cast<const uint4*>(&h[word]);
                c[0] = q4.w, c[1] = q4.z, c[2] = q4.y, c[3] = q4.x;
            } else {
                for (int r0 = 0; r0 < CL; r0 += 4) {
                    uint4 q4[4];
#pragma unroll
                    for (int j = 0; j < 4; j++)
                        q4[j] = r0 + j < CL ? *reinterpret_cast<const uint4*>(cluster.map_shared_rank(h, r0 + j) + word) : make_uint4(0, 0, 0, 0);
#pragma unroll
                    for (int j = 0; j < 4; j++) c[0] += q4[j].w, c[1] += q4[j].z, c[2] += q4[j].y, c[3] += q4[j].x;
                }
            }
        }
        if (pass == 1) {   // the other buffer (read by the cluster before this pass's barrier) is refilled in pass 2
            hist[0][2 * t] = 0;
            hist[0][2 * t + 1] = 0;
        }
        if (pass == 1) trace_last(p.ctl.trace, 6);
        const uint32_t s = c[0] + c[1] + c[2] + c[3], incl = warp_incl_scan(s, lane);
        if (lane == 31) wsum[warp] = incl;
        __syncthreads();
        const uint32_t ws = warp_incl_scan(wsum[lane], lane);
        const uint32_t wbase = __shfl_sync(0xffffffffu, ws, (warp + 31) & 31);
        uint32_t above = (warp ? wbase : 0u) + incl - s;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            if (above < k && above + c[j] >= k) {
                sel[0] = uint32_t(nb - 1 - 4 * t - j);
                sel[1] = above;
            }
            above += c[j];
        }
        __syncthreads();
        prefix |= sel[0] << shift;
        mask |= uint32_t(nb - 1) << shift;
        k -= sel[1];
        if (pass == 1) trace_last(p.ctl.trace, 7);
    }
    trace_last(p.ctl.trace, 2);
    // prefix is the TOPK-th largest pattern; every key above it, then the first k equal to it, in key order.
    // Lane i keeps round i's ballots, so the counts and the writes below cost a few instructions a warp.
    uint32_t mybg = 0, mybe = 0;
#pragma unroll
    for (int i = 0; i < ITEMS; i++) {
        const bool ok = 32 * i < lim;
        const uint32_t bg = __ballot_sync(0xffffffffu, ok && v[i] > prefix);
        const uint32_t be = __ballot_sync(0xffffffffu, ok && v[i] == prefix);
        if (lane == i) {
            mybg = bg;
            mybe = be;
        }
    }
    const uint32_t cg_incl = warp_incl_scan(uint32_t(__popc(mybg)), lane);
    const uint32_t ce_incl = warp_incl_scan(uint32_t(__popc(mybe)), lane);
    // every warp's counts go to every CTA of the cluster (pushed again), so that the offsets below are local arithmetic
    if (SINGLE) {
        if (lane == 31) {
            wall[0][0][warp] = cg_incl;
            wall[1][0][warp] = ce_incl;
        }
        __syncthreads();
    } else {
        const uint32_t gcount = __shfl_sync(0xffffffffu, cg_incl, 31), ecount = __shfl_sync(0xffffffffu, ce_incl, 31);
        if (lane < CL) {   // lane r writes this warp's two counts into CTA r
            cluster_st_u32(cluster_map(wall_here + uint32_t((0 * 8 + rank) * SEL_WARPS + warp) * 4u, uint32_t(lane)), gcount);
            cluster_st_u32(cluster_map(wall_here + uint32_t((1 * 8 + rank) * SEL_WARPS + warp) * 4u, uint32_t(lane)), ecount);
        }
        cluster_arrive();
        cluster_wait();
    }
    // offsets of this CTA's warps: everything counted by lower ranks, then this CTA's lower warps
    if (warp < 2) {
        uint32_t before = 0, all = 0;
        for (int r = 0; r < CL; r++) {
            uint32_t sum = wall[warp][r][lane];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            if (r < rank) before += sum;
            all += sum;
        }
        const uint32_t mine = wall[warp][rank][lane];
        base[warp][lane] = before + warp_incl_scan(mine, lane) - mine;
        if (lane == 0) base[warp][SEL_WARPS] = all;
    }
    __syncthreads();
    {
        // lane i writes round i's keys: bit l of its ballot is key w0 + 32 i + l
        const uint32_t ngt = base[0][SEL_WARPS];
        uint32_t gpos = base[0][warp] + cg_incl - uint32_t(__popc(mybg));
        uint32_t epos = base[1][warp] + ce_incl - uint32_t(__popc(mybe));
        const uint32_t j0 = uint32_t(w0 + 32 * lane);
        while (mybg) {
            const int l = __ffs(mybg) - 1;
            mybg &= mybg - 1;
            out[gpos++] = j0 + l;
        }
        while (mybe && epos < k) {
            const int l = __ffs(mybe) - 1;
            mybe &= mybe - 1;
            out[ngt + epos++] = j0 + l;
        }
        if (rank == 0)
            for (int j = t; j < EMBLA_RECENT; j += SEL_T) out[EMBLA_TOPK + j] = uint32_t(n + j);
    }
    // (the last loads from another CTA's shared memory, the third pass's, were complete before the barrier above, and every
    // push into it too: a CTA may leave at once)
    trace_last(p.ctl.trace, 3);
}

template <int ITEMS, bool BULK, bool SINGLE>
static cudaError_t launch_select_kernel(const SelectParams& p, int batch, int cl, int device, bool pdl, cudaStream_t s) {
    const size_t smem = BULK ? size_t(SEL_T) * ITEMS * 4 : 0;
    static bool configured[64] = {};
    if (smem > 0 && !configured[device & 63]) {
        cudaError_t e = cudaFuncSetAttribute(select_keys_kernel<ITEMS, BULK, SINGLE>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return e;
        configured[device & 63] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.n_kv_heads * cl, batch);
    cfg.blockDim = dim3(SEL_T);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = cl;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = 1;
    // without a cluster only the dependent-launch attribute (the second entry) applies
    cfg.attrs = SINGLE ? at + 1 : at;
    cfg.numAttrs = (SINGLE ? 0 : 1) + (pdl ? 1 : 0);
    return cudaLaunchKernelEx(&cfg, select_keys_kernel<ITEMS, BULK, SINGLE>, p);
}

template <int ITEMS, bool BULK>
static cudaError_t launch_select(const SelectParams& p, int batch, int cl, int device, bool pdl, cudaStream_t s) {
    return cl == 1 ? launch_select_kernel<ITEMS, BULK, true>(p, batch, cl, device, pdl, s)
                   : launch_select_kernel<ITEMS, BULK, false>(p, batch, cl, device, pdl, s);
}

template <bool BULK>
static cudaError_t launch_select_items(const SelectParams& p, int per_thread, int batch, int cl, int device, bool pdl, cudaStream_t s) {
    if (per_thread <= 1) return launch_select<1, BULK>(p, batch, cl, device, pdl, s);
    if (per_thread <= 2) return launch_select<2, BULK>(p, batch, cl, device, pdl, s);
    if (per_thread <= 4) return launch_select<4, BULK>(p, batch, cl, device, pdl, s);
    if (per_thread <= 8) return launch_select<8, BULK>(p, batch, cl, device, pdl, s);
    if (per_thread <= 16) return launch_select<16, BULK>(p, batch, cl, device, pdl, s);
    return launch_select<32, BULK>(p, batch, cl, device, pdl, s);
}

}  // namespace embla

using namespace embla;

extern "C" EmblaStatus embla_select_keys(EmblaAttn* ctx, const float* scores_dev, int64_t scores_stride,
                                         const int32_t* seq_lens_dev, int32_t batch, int32_t max_seq_len,
                                         uint32_t* idx_dev, void* stream) {
    if (!ctx || !scores_dev || !seq_lens_dev || !idx_dev) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_select_keys: null argument");
    EMBLA_CHECK_DEVICE("embla_select_keys", ctx, static_cast<const EmblaKVPool*>(nullptr));
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
    p.ctl = kernel_ctl(ctx);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int n_max = max_len - EMBLA_RECENT;   // keys a pair ranks: CL CTAs x 1024 threads x ITEMS
    if (n_max > EMBLA_SELECT_MAX_KEYS - EMBLA_RECENT)
        EMBLA_FAIL(EMBLA_UNSUPPORTED, "embla_select_keys: %d keys (at most %d: 8 CTAs x 1024 threads x 32 keys + the %d latest)", max_len,
                   EMBLA_SELECT_MAX_KEYS, EMBLA_RECENT);
    // long rows: as many CTAs a pair as it takes to hold its keys in registers (32 a lane); small batches: a cluster of
    // 2, 4 or 8 CTAs per (sequence, kv head), as many as keep the GPU busy
    int cl = 1;
    while (cl < 8 && n_max > 1024 * 32 * cl) cl *= 2;
    while (cl < 8 && 2 * cl * p.n_kv_heads * batch <= ctx->sm_count && n_max > 1024 * cl) cl *= 2;
    const int per_thread = (n_max + 1024 * cl - 1) / (1024 * cl);
    // bulk copies want 16-byte aligned rows; any other layout takes the lanes' own loads
    const bool bulk = reinterpret_cast<uintptr_t>(scores_dev) % 16 == 0 && scores_stride % 4 == 0;
    const cudaError_t e = bulk ? launch_select_items<true>(p, per_thread, batch, cl, ctx->device, ctx->pdl != 0, s)
                               : launch_select_items<false>(p, per_thread, batch, cl, ctx->device, ctx->pdl != 0, s);
    EMBLA_CUDA_TRY(e);
    EMBLA_CUDA_TRY(cudaGetLastError());
    return EMBLA_OK;
}
