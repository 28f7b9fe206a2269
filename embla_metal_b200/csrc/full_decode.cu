// Decode attention of the full layers: ReLU² over the int8 paged cache, one query token per
// sequence. Replaces attn_full8 (Sources/EmblaMetal/Kernels/attention.metal:235-363; its dispatch
// Sources/EmblaMetal/Engine.swift:796-818).
//
// The kernel is bound by HBM: every key costs 2 x 128 code bytes + 2 scales, used once. Design:
//  * grid (split, kv head, sequence); a CTA streams a contiguous range of the sequence's
//    128-position pages through a ring of shared-memory stages filled by TMA (one 2-D tiled copy of
//    the page's 256 code rows with the 128-byte swizzle + one bulk copy of its scales), issued by a
//    producer warp; 4 consumer warps each take 32 of a page's 128 keys.
//  * q·k and w·v run as warp-level m16n8k16 tensor-core tiles on fp16: the int8 codes are exact in
//    fp16 and are widened in registers; the query heads of the kv head are the M rows (<= 8 used),
//    keys are N for S = Q Kᵀ and K for O = P V, so S's accumulators are P's A fragments.
//    fp32 CUDA-core math could not keep up with the bytes (4 heads x 256 FMAs per 260 bytes).
//  * split partial sums go to scratch; the last CTA of a (sequence, kv head) to arrive adds them in
//    split order (ReLU² partials just add, attention.metal:143-145) — deterministic, one launch.
//  * SCORES: each consumer thread also takes one key of the page and computes the kv head's query
//    heads' dots as one fp32 fmaf chain over d = 0..127 (the summation order the CPU oracle fixes),
//    so the selection that follows is reproducible bit for bit.
#include "common.cuh"

namespace embla {

constexpr int FD_CONSUMERS = 4;
constexpr int FD_THREADS = (FD_CONSUMERS + 1) * 32;
constexpr int FD_STAGE_BYTES = 2 * CODE_BYTES + 1024;   // codes + K and V scales (fp32 at most)
constexpr int FD_PART = HD + 4;                         // floats per (split, head): 128 sums, sum of weights

struct FullDecodeParams {
    const uint8_t* pool;
    const int32_t* block_table;
    const int32_t* seq_lens;
    const void* q;
    const void* g1;
    const void* g2;
    void* o;
    float* partials;
    int* counters;
    int* err;
    float* scores;
    int64_t q_stride, o_stride, scores_stride;
    size_t page_bytes;
    int table_stride, layer, n_layers, n_kv_heads, G, scale_bytes, rows_per_page, nsplit, prenormed, ng;
};

// Row of the 8-key tile that MMA column g of S = Q Kᵀ stands for. Chosen so that both the K loads
// (thread (g, c): row rho(g), chunks c and c + 4) and the V loads (thread (g, c): rows rho(2c),
// rho(2c + 1), chunk g) hit 8 different 16-byte bank groups per quarter warp under the swizzle
// chunk ^ (row % 8).
__device__ __forceinline__ int rho(int g) {
    const int h = g >> 1, base = h < 2 ? 2 * h : 2 * h + 1;
    return base ^ ((g & 1) << 2);
}

template <int DT>
__device__ __forceinline__ void prep_query_smem(const FullDecodeParams& p, int b, int kvh, __half (*qh)[HD], float (*qf)[HD],
                                                int warp, int lane, int nwarps) {
    // Heads of this kv head into shared memory as fp16 (and fp32 for the scoring chain): optional
    // head norm with gains in the oracle's operation order, rounded to the activation dtype.
    for (int g = warp; g < 8; g += nwarps) {
        float x[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (g < p.G) {
            const size_t off = size_t(b) * p.q_stride + size_t(kvh * p.G + g) * HD;
#pragma unroll
            for (int i = 0; i < 4; i++) x[i] = Act<DT>::load(p.q, off + lane + 32 * i);
            if (!p.prenormed) {
                float ss = 0.0f;
#pragma unroll
                for (int i = 0; i < 4; i++) ss = __fadd_rn(ss, __fmul_rn(x[i], x[i]));
                float tot = 0.0f;
                for (int l = 0; l < 32; l++) tot = __fadd_rn(tot, __shfl_sync(0xffffffffu, ss, l));
                const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, float(HD)), EPS32)));
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int d = lane + 32 * i;
                    float gn = r;
                    if (p.ng >= 1) gn = __fmul_rn(gn, __fadd_rn(1.0f, Act<DT>::load(p.g1, d)));
                    if (p.ng >= 2) gn = __fmul_rn(gn, __fadd_rn(1.0f, Act<DT>::load(p.g2, d)));
                    x[i] = Act<DT>::round(__fmul_rn(x[i], gn));
                }
            }
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            qh[g][lane + 32 * i] = __float2half_rn(x[i]);
            if (qf) qf[g][lane + 32 * i] = x[i];
        }
    }
}

template <int DT, int STAGES, bool SCORES>
__global__ void __launch_bounds__(FD_THREADS) full_decode_kernel(const __grid_constant__ CUtensorMap tmap,
                                                                const FullDecodeParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* stages = smem;
    __half(*qh)[HD] = reinterpret_cast<__half(*)[HD]>(smem + STAGES * FD_STAGE_BYTES);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * FD_STAGE_BYTES + 8 * HD * 2);
    uint64_t* empty = full + STAGES;
    float(*qf)[HD] = SCORES ? reinterpret_cast<float(*)[HD]>(empty + STAGES) : nullptr;
    __shared__ int s_last, s_failed, s_issued;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int S = p.seq_lens[b];
    const int npages = (S + BLK - 1) / BLK;
    const int pps = (npages + p.nsplit - 1) / p.nsplit;
    const int pg0 = split * pps;
    const int n = max(0, min(npages, pg0 + pps) - pg0);

    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], FD_CONSUMERS);
        }
        s_failed = 0;
        s_issued = 0;
        fence_barrier_init();
    }
    prep_query_smem<DT>(p, b, kvh, qh, qf, warp, lane, FD_CONSUMERS + 1);
    __syncthreads();

    const int g = lane >> 2, c = lane & 3;
    float O[16][4];
#pragma unroll
    for (int i = 0; i < 16; i++) O[i][0] = O[i][1] = O[i][2] = O[i][3] = 0.0f;
    float psum = 0.0f;

    if (warp == FD_CONSUMERS) {
        // ---- producer: one lane keeps the ring of stages full
        if (lane == 0) {
            const uint32_t tx = 2 * CODE_BYTES + 2 * BLK * p.scale_bytes;
            for (int i = 0; i < n; i++) {
                const int st = i % STAGES, use = i / STAGES;
                if (use > 0 && !mbar_wait_bounded(&empty[st], (use - 1) & 1)) {
                    atomicExch(p.err, ERR_WAIT_EMPTY);
                    break;
                }
                const int block = p.block_table[size_t(b) * p.table_stride + pg0 + i];
                const long page = (long(block) * p.n_layers + p.layer) * p.n_kv_heads + kvh;
                uint8_t* dst = stages + st * FD_STAGE_BYTES;
                mbar_expect_tx(&full[st], tx);
                tma_load_2d(dst, &tmap, 0, int(page * p.rows_per_page), &full[st]);
                bulk_load_1d(dst + 2 * CODE_BYTES, p.pool + size_t(page) * p.page_bytes + 2 * CODE_BYTES,
                             2 * BLK * p.scale_bytes, &full[st]);
                *reinterpret_cast<volatile int*>(&s_issued) = i + 1;
            }
        }
    } else {
        // ---- consumers
        uint32_t qa0[8], qa2[8];
#pragma unroll
        for (int t = 0; t < 8; t++) {
            const int d0 = (t < 4) ? 16 * c + 4 * t : 64 + 16 * c + 4 * (t - 4);
            qa0[t] = *reinterpret_cast<const uint32_t*>(&qh[g][d0]);
            qa2[t] = *reinterpret_cast<const uint32_t*>(&qh[g][d0 + 2]);
        }
        const int rho_g = rho(g), kA = rho(2 * c), kB = kA ^ 4;
        const float scale = rsqrtf(float(HD));
        for (int i = 0; i < n; i++) {
            const int st = i % STAGES, use = i / STAGES;
            if (!mbar_wait_bounded(&full[st], use & 1)) {
                atomicExch(p.err, ERR_WAIT_FULL);
                *reinterpret_cast<volatile int*>(&s_failed) = 1;
                break;
            }
            const uint8_t* Kb = stages + st * FD_STAGE_BYTES;
            const uint8_t* Vb = Kb + CODE_BYTES;
            const uint8_t* ksc = Kb + 2 * CODE_BYTES;
            const uint8_t* vsc = ksc + BLK * p.scale_bytes;
            const int key_base = (pg0 + i) * BLK;

            if (SCORES) {
                // one key a thread: the kv head's heads' dots as one fmaf chain over d ascending
                const int r = warp * 32 + lane;
                if (key_base + r < S) {
                    float dot[8];
#pragma unroll
                    for (int h = 0; h < 8; h++) dot[h] = 0.0f;
                    const uint8_t* krow = Kb + r * 128;
#pragma unroll
                    for (int ch = 0; ch < 8; ch++) {
                        const uint4 w4 = *reinterpret_cast<const uint4*>(krow + ((ch ^ (r & 7)) << 4));
                        const uint32_t w[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
                        for (int e = 0; e < 16; e++) {
                            const float kv = float(int(int8_t((w[e >> 2] >> (8 * (e & 3))) & 0xff)));
                            const int d = ch * 16 + e;
#pragma unroll
                            for (int h = 0; h < 8; h++)
                                if (h < p.G) dot[h] = __fmaf_rn(qf[h][d], kv, dot[h]);
                        }
                    }
                    const float ks = load_scale(ksc, r, p.scale_bytes);
                    float best = __fmul_rn(dot[0], ks);
#pragma unroll
                    for (int h = 1; h < 8; h++) {
                        if (h < p.G) {
                            const float t = __fmul_rn(dot[h], ks);
                            if (t > best) best = t;
                        }
                    }
                    p.scores[(size_t(b) * p.n_kv_heads + kvh) * p.scores_stride + key_base + r] = best;
                }
            }

#pragma unroll
            for (int step = 0; step < 2; step++) {
                const int R0 = warp * 32 + step * 16;
                float pw[2][2];
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    const int r = R0 + 8 * j + rho_g;
                    const uint8_t* krow = Kb + r * 128;
                    const uint4 lo = *reinterpret_cast<const uint4*>(krow + ((c ^ rho_g) << 4));
                    const uint4 hi = *reinterpret_cast<const uint4*>(krow + (((c + 4) ^ rho_g) << 4));
                    const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
                    float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                    for (int t = 0; t < 8; t++) {
                        const uint32_t x = w[t] ^ 0x80808080u;
                        mma_16816(s, qa0[t], 0u, qa2[t], 0u, h2_from_biased_bytes(x, 0x4140), h2_from_biased_bytes(x, 0x4342));
                    }
                    const int keyA = R0 + 8 * j + kA, keyB = R0 + 8 * j + kB;
                    const float tA = s[0] * load_scale(ksc, keyA, p.scale_bytes);
                    const float tB = s[1] * load_scale(ksc, keyB, p.scale_bytes);
                    const float aA = fmaxf(tA * scale, 0.0f), aB = fmaxf(tB * scale, 0.0f);
                    const float wA = (key_base + keyA < S) ? aA * aA : 0.0f;
                    const float wB = (key_base + keyB < S) ? aB * aB : 0.0f;
                    psum += wA + wB;
                    pw[j][0] = wA != 0.0f ? wA * load_scale(vsc, keyA, p.scale_bytes) : 0.0f;
                    pw[j][1] = wB != 0.0f ? wB * load_scale(vsc, keyB, p.scale_bytes) : 0.0f;
                }
                // V-skip: a 16-key tile whose weights are all zero adds nothing (attention.metal:310)
                const bool live = pw[0][0] != 0.0f || pw[0][1] != 0.0f || pw[1][0] != 0.0f || pw[1][1] != 0.0f;
                if (!__any_sync(0xffffffffu, live)) continue;
                const uint32_t pa0 = pack_h2(pw[0][0], pw[0][1]), pa2 = pack_h2(pw[1][0], pw[1][1]);
                const uint8_t* vA = Vb + (R0 + kA) * 128 + ((g ^ kA) << 4);
                const uint8_t* vB = Vb + (R0 + kB) * 128 + ((g ^ kB) << 4);
                const uint4 a4 = *reinterpret_cast<const uint4*>(vA);
                const uint4 b4 = *reinterpret_cast<const uint4*>(vB);
                const uint4 c4 = *reinterpret_cast<const uint4*>(vA + 8 * 128);
                const uint4 d4 = *reinterpret_cast<const uint4*>(vB + 8 * 128);
                const uint32_t va[4] = {a4.x, a4.y, a4.z, a4.w}, vb[4] = {b4.x, b4.y, b4.z, b4.w};
                const uint32_t vc[4] = {c4.x, c4.y, c4.z, c4.w}, vd[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
                for (int wq = 0; wq < 4; wq++) {
                    const uint32_t x = va[wq] ^ 0x80808080u, y = vb[wq] ^ 0x80808080u;
                    const uint32_t x2 = vc[wq] ^ 0x80808080u, y2 = vd[wq] ^ 0x80808080u;
                    const uint32_t z0 = __byte_perm(x, y, 0x5140), z1 = __byte_perm(x, y, 0x7362);
                    const uint32_t u0 = __byte_perm(x2, y2, 0x5140), u1 = __byte_perm(x2, y2, 0x7362);
                    mma_16816(O[4 * wq + 0], pa0, 0u, pa2, 0u, h2_from_biased_bytes(z0, 0x4140), h2_from_biased_bytes(u0, 0x4140));
                    mma_16816(O[4 * wq + 1], pa0, 0u, pa2, 0u, h2_from_biased_bytes(z0, 0x4342), h2_from_biased_bytes(u0, 0x4342));
                    mma_16816(O[4 * wq + 2], pa0, 0u, pa2, 0u, h2_from_biased_bytes(z1, 0x4140), h2_from_biased_bytes(u1, 0x4140));
                    mma_16816(O[4 * wq + 3], pa0, 0u, pa2, 0u, h2_from_biased_bytes(z1, 0x4342), h2_from_biased_bytes(u1, 0x4342));
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[st]);
        }
    }

    // ---- the 4 consumer warps' sums into one partial (the stage ring is free now: every page that
    // was requested has been waited for, unless a wait gave up — then drain what is still in flight)
    __syncthreads();
    if (s_failed) {
        if (tid == 0) {
            for (int i = max(0, s_issued - STAGES); i < s_issued; i++)
                if (!mbar_wait_bounded(&full[i % STAGES], (i / STAGES) & 1)) atomicExch(p.err, ERR_WAIT_DRAIN);
        }
        __syncthreads();
    }
    float(*red)[8][HD] = reinterpret_cast<float(*)[8][HD]>(stages);
    float(*redp)[8] = reinterpret_cast<float(*)[8]>(stages + FD_CONSUMERS * 8 * HD * 4);
    if (warp < FD_CONSUMERS) {
        psum += __shfl_xor_sync(0xffffffffu, psum, 1);
        psum += __shfl_xor_sync(0xffffffffu, psum, 2);
#pragma unroll
        for (int i = 0; i < 16; i++) {
            red[warp][g][32 * c + i] = O[i][0];
            red[warp][g][32 * c + 16 + i] = O[i][1];
        }
        if (c == 0) redp[warp][g] = psum;
    }
    __syncthreads();

    const int pair = b * p.n_kv_heads + kvh;
    const float sink = sqrtf(float(HD));
    if (p.nsplit == 1) {
        for (int idx = tid; idx < p.G * HD; idx += FD_THREADS) {
            const int hh = idx >> 7, d = idx & 127;
            const float num = ((red[0][hh][d] + red[1][hh][d]) + red[2][hh][d]) + red[3][hh][d];
            const float den = sink + (((redp[0][hh] + redp[1][hh]) + redp[2][hh]) + redp[3][hh]);
            Act<DT>::store(p.o, size_t(b) * p.o_stride + size_t(kvh * p.G + hh) * HD + d, num / den);
        }
        return;
    }
    float* part = p.partials + (size_t(pair) * p.nsplit + split) * p.G * FD_PART;
    for (int idx = tid; idx < p.G * HD; idx += FD_THREADS) {
        const int hh = idx >> 7, d = idx & 127;
        part[hh * FD_PART + d] = ((red[0][hh][d] + red[1][hh][d]) + red[2][hh][d]) + red[3][hh][d];
        if (d == 0) part[hh * FD_PART + HD] = ((redp[0][hh] + redp[1][hh]) + redp[2][hh]) + redp[3][hh];
    }
    // last CTA of the pair to arrive adds the splits in order (arrive_last, common.metal:88-99)
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const int prev = atomicAdd(&p.counters[pair], 1);
        s_last = prev == p.nsplit - 1;
        if (s_last) p.counters[pair] = 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const float* base = p.partials + size_t(pair) * p.nsplit * p.G * FD_PART;
    for (int idx = tid; idx < p.G * HD; idx += FD_THREADS) {
        const int hh = idx >> 7, d = idx & 127;
        float num = 0.0f, den = sink;
        for (int s = 0; s < p.nsplit; s++) {
            const float* q2 = base + (size_t(s) * p.G + hh) * FD_PART;
            den += __ldcg(q2 + HD);
            num += __ldcg(q2 + d);
        }
        Act<DT>::store(p.o, size_t(b) * p.o_stride + size_t(kvh * p.G + hh) * HD + d, num / den);
    }
}

template <int STAGES, bool SCORES>
constexpr size_t fd_smem_bytes() {
    return 1024 + size_t(STAGES) * FD_STAGE_BYTES + 8 * HD * 2 + 2 * STAGES * 8 + (SCORES ? 8 * HD * 4 : 0);
}

// Key ranges per (sequence, kv head): fill `slots` resident CTAs in whole waves, with ranges long
// enough to amortise a CTA's start-up (the reference's chunks8, Engine.swift:737-740, for 148 SMs).
int choose_splits(int pairs, int pages, int slots, int max_slots) {
    int best = 1;
    double best_cost = 1e30;
    const int limit = max(1, min(pages, max_slots / max(pairs, 1)));
    for (int ns = 1; ns <= limit; ns++) {
        const long ctas = long(pairs) * ns;
        const long waves = (ctas + slots - 1) / slots;
        const int per = (pages + ns - 1) / ns;
        const double cost = double(waves) * (per + 3.0);   // 3 pages' worth of start-up and combine per CTA
        if (cost < best_cost - 1e-9) {
            best_cost = cost;
            best = ns;
        }
    }
    return best;
}

}  // namespace embla

using namespace embla;

template <int DT, bool SCORES>
static EmblaStatus launch_full_decode(EmblaAttn* ctx, const EmblaKVPool* pool, const FullDecodeParams& p, int batch,
                                      cudaStream_t s) {
    constexpr int STAGES = 3;
    constexpr size_t smem = fd_smem_bytes<STAGES, SCORES>();
    auto kern = full_decode_kernel<DT, STAGES, SCORES>;
    static bool configured[64] = {};   // per instantiation and device
    if (!configured[ctx->device & 63]) {
        EMBLA_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        configured[ctx->device & 63] = true;
    }
    dim3 grid(p.nsplit, p.n_kv_heads, batch);
    kern<<<grid, FD_THREADS, smem, s>>>(pool->tmap_codes, p);
    EMBLA_CUDA_TRY(cudaGetLastError());
    return EMBLA_OK;
}

extern "C" EmblaStatus embla_attn_full_decode(EmblaAttn* ctx, const EmblaKVPool* pool, const EmblaKVView* view,
                                              const EmblaQuery* q, void* o_dev, int64_t o_stride,
                                              float* scores_dev, int64_t scores_stride, void* stream) {
    if (!ctx || !pool || !view || !q || !o_dev) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_full_decode: null argument");
    if (pool->kv_dtype != EMBLA_KV_INT8) EMBLA_FAIL(EMBLA_UNSUPPORTED, "embla_attn_full_decode: the pool is not int8");
    if (pool->n_kv_heads != ctx->cfg.n_kv_heads)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_full_decode: pool has %d kv heads, context %d", pool->n_kv_heads,
                   ctx->cfg.n_kv_heads);
    if (view->layer < 0 || view->layer >= pool->n_layers)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_full_decode: layer %d outside the pool's %d", view->layer, pool->n_layers);
    if (view->batch <= 0 || view->batch > ctx->cfg.max_batch)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_full_decode: batch %d outside 1..%d", view->batch, ctx->cfg.max_batch);
    if (!view->block_table_dev || !view->seq_lens_dev || !q->q_dev)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_full_decode: null block table, seq_lens or q");
    if (!q->prenormed && ((q->ng >= 1 && !q->g1_dev) || (q->ng >= 2 && !q->g2_dev) || q->ng < 0 || q->ng > 2))
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_full_decode: ng %d without its gain vectors", q->ng);
    const int max_len = view->max_seq_len > 0 ? view->max_seq_len : ctx->cfg.max_context;
    if (max_len > ctx->cfg.max_context)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_full_decode: max_seq_len %d over the context's %d", max_len, ctx->cfg.max_context);

    FullDecodeParams p;
    p.pool = pool->base;
    p.block_table = view->block_table_dev;
    p.seq_lens = view->seq_lens_dev;
    p.q = q->q_dev;
    p.g1 = q->g1_dev;
    p.g2 = q->g2_dev;
    p.o = o_dev;
    p.partials = ctx->partials;
    p.counters = ctx->counters;
    p.err = ctx->err_dev;
    p.scores = scores_dev;
    p.q_stride = q->q_stride;
    p.o_stride = o_stride;
    p.scores_stride = scores_stride;
    p.page_bytes = pool->page_bytes;
    p.table_stride = view->table_stride;
    p.layer = view->layer;
    p.n_layers = pool->n_layers;
    p.n_kv_heads = pool->n_kv_heads;
    p.G = ctx->cfg.n_q_heads / ctx->cfg.n_kv_heads;
    p.scale_bytes = pool->scale_bytes;
    p.rows_per_page = pool->rows_per_page;
    p.prenormed = q->prenormed;
    p.ng = q->ng;
    const int pairs = view->batch * pool->n_kv_heads;
    const int pages = (max_len + BLK - 1) / BLK;
    p.nsplit = choose_splits(pairs, pages, 2 * ctx->sm_count, ctx->partial_slots);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool bf = ctx->cfg.act_dtype == EMBLA_BF16;
    if (scores_dev) {
        return bf ? launch_full_decode<EMBLA_BF16, true>(ctx, pool, p, view->batch, s)
                  : launch_full_decode<EMBLA_F16, true>(ctx, pool, p, view->batch, s);
    }
    return bf ? launch_full_decode<EMBLA_BF16, false>(ctx, pool, p, view->batch, s)
              : launch_full_decode<EMBLA_F16, false>(ctx, pool, p, view->batch, s);
}
