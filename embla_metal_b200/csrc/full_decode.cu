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
#include <cstdlib>

#include "kv_row.cuh"

namespace embla {

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
    KernelCtl ctl;
    float* scores;
    int64_t q_stride, o_stride, scores_stride;
    size_t page_bytes;
    int table_stride, layer, n_layers, n_kv_heads, G, scale_bytes, rows_per_page, nsplit, prenormed, ng;
    // the current token's raw k and v rows, or NULL: appended by this launch (kv_append fused, attention.metal:113-140)
    const void* k_new;
    const void* v_new;
    int64_t kv_stride;
    int norm_k;
};

// Row of the 8-key tile that MMA column g of S = Q Kᵀ stands for. Chosen so that both the K loads
// (thread (g, c): row rho(g), chunks c and c + 4) and the V loads (thread (g, c): rows rho(2c),
// rho(2c + 1), chunk g) hit 8 different 16-byte bank groups per quarter warp under the swizzle
// chunk ^ (row % 8).
__device__ __forceinline__ int rho(int g) {
    const int h = g >> 1, base = h < 2 ? 2 * h : 2 * h + 1;
    return base ^ ((g & 1) << 2);
}

// 8x8 b16 transpose across the warp: lane (g, c) gives row g, columns 2c, 2c+1 and receives row g,
// columns 2c, 2c+1 of the transpose.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
    uint32_t r;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(x));
    return r;
}

template <int SB>
__device__ __forceinline__ float ld_scale(const uint8_t* p, int i) {
    if (SB == 4) return reinterpret_cast<const float*>(p)[i];
    return __half2float(reinterpret_cast<const __half*>(p)[i]);
}

// int8 code (already ^0x80, byte `k` of x) -> fp32, exactly: 2^23 + 128 + code, minus 2^23 + 128.
__device__ __forceinline__ float f32_from_biased_byte(uint32_t x, int k) {
    return __fadd_rn(__uint_as_float(__byte_perm(x, 0x4B000000u, 0x7440 | k)), -8388736.0f);
}

constexpr int QF_LD = HD + 4;   // fp32 query rows padded so that two heads never share a bank
// where the cluster inbox starts in the (1024-byte aligned) dynamic shared memory: behind stages, queries and barriers
__host__ __device__ constexpr size_t fd_inbox_offset(int stages, bool scores) {
    return ((size_t(stages) * FD_STAGE_BYTES + 8 * HD * 2 + 2 * size_t(stages) * 8 + (scores ? 8 * QF_LD * 4 : 0)) + 15) / 16 * 16;
}

// acc = fma(q.lo, k.lo, acc); acc = fma(q.hi, k.hi, acc) on packed fp16 pairs: products exact, each step rounded
// once to fp32 (the mixed-precision fma of sm_100).
__device__ __forceinline__ void fma_pair_f16(float& acc, uint32_t k, uint32_t q) {
    asm("{\n .reg .b16 kl, kh, ql, qh;\n mov.b32 {kl, kh}, %1;\n mov.b32 {ql, qh}, %2;\n"
        " fma.rn.f32.f16 %0, ql, kl, %0;\n fma.rn.f32.f16 %0, qh, kh, %0;\n}\n"
        : "+f"(acc)
        : "r"(k), "r"(q));
}

// SG: 0 = no scores; 1, 2, 4, 8 = also the key scores, for that many query heads a kv head; 9 = scores for any
// head count up to 8 (the count read at run time).
// NCONS consumer warps share the keys of every page for the attention; with scores, 4 more warps (one key a thread)
// compute the key scores from the same stage; the last warp is the producer.
// CL: the key ranges of a pair are the CTAs of one thread-block cluster (at most 4), launched as such; every range sends
// its partial rows, head by head, into the shared memory of the CTA that finishes that head (head h: CTA h % ranges), so
// the combine needs one cluster barrier and no global scratch.
template <int DT, int SB, int NCONS, int STAGES, int SG, bool CL>
__global__ void __launch_bounds__((NCONS + (SG != 0 ? 4 : 0) + 1) * 32, 2)   // two CTAs an SM: at most 112 registers a thread
    full_decode_kernel(const __grid_constant__ CUtensorMap tmap, const FullDecodeParams p) {
    constexpr bool SCORES = SG != 0;
    constexpr int GT = SG == 9 ? 8 : SG;
    constexpr int NSC = SCORES ? 4 : 0;            // scoring warps
    constexpr int NWORK = NCONS + NSC;             // warps that read the stages
    constexpr int THREADS = (NWORK + 1) * 32;
    constexpr int KPW = BLK / NCONS;   // keys of a page per consumer warp
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* stages = smem;
    __half(*qh)[HD] = reinterpret_cast<__half(*)[HD]>(smem + STAGES * FD_STAGE_BYTES);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * FD_STAGE_BYTES + 8 * HD * 2);
    uint64_t* empty = full + STAGES;
    float(*qf)[QF_LD] = reinterpret_cast<float(*)[QF_LD]>(empty + STAGES);   // SCORES only
    __shared__ int s_last, s_failed, s_issued;
    __shared__ uint64_t patched;   // the appended row is in the staged copy of the last page

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    trace_first(p.ctl.trace, 0);
    // Launched with the dependent-launch attribute, the kernel ahead of this one in the stream may still be running
    // here. An "early" launch (the step driver knows that kernel writes none of this layer's pages) starts its first
    // pages before it waits for that kernel; seq_lens and the block table are inputs of the whole step.
    const int S = p.seq_lens[b];   // (an input of the whole step: read ahead of the wait, its latency hidden behind it)
    if (!p.ctl.early) {
        pdl_wait();
        pdl_launch_dependents();
    }
    const int npages = (S + BLK - 1) / BLK;
    const int pps = (npages + p.nsplit - 1) / p.nsplit;
    const int pg0 = split * pps;
    const int n = max(0, min(npages, pg0 + pps) - pg0);
    // The CTA whose range ends with the sequence's last page also appends the current token (position S - 1): its
    // producer warp quantises the k and v rows, writes them to the page for the steps to come and, because the page
    // may have been fetched before that write, puts them into the staged copy before the consumers read it.
    const bool appends = p.k_new != nullptr && n > 0 && pg0 + n == npages;

    // ---- producer: one lane keeps the ring of stages full
    const uint32_t tx = 2 * CODE_BYTES + 2 * BLK * SB;
    // `block`: the page's physical block if the caller has it already, else -1 (read from the table here)
    auto issue = [&](int i, int block) {
        const int st = i % STAGES, use = i / STAGES;
        if (i == p.ctl.stall_at) return false;   // diagnostic stall: the consumers' wait for this page runs out
        if (use > 0 && !mbar_wait_bounded(p.ctl.wait_cycles, &empty[st], (use - 1) & 1)) {
            atomicExch(p.ctl.err, ERR_WAIT_EMPTY);
            return false;
        }
        if (block < 0) block = p.block_table[size_t(b) * p.table_stride + pg0 + i];
        const long page = (long(block) * p.n_layers + p.layer) * p.n_kv_heads + kvh;
        uint8_t* dst = stages + st * FD_STAGE_BYTES;
        mbar_expect_tx(&full[st], tx);
        tma_load_2d(dst, &tmap, 0, int(page * p.rows_per_page), &full[st]);
        bulk_load_1d(dst + 2 * CODE_BYTES, p.pool + size_t(page) * p.page_bytes + 2 * CODE_BYTES, 2 * BLK * SB, &full[st]);
        *reinterpret_cast<volatile int*>(&s_issued) = i + 1;
        return true;
    };
    int next = 0;
    bool issuing = true;
    if (warp == NWORK) {
        // The producer warp starts before anyone else: lane i looks up the block of the range's page i (the lookups in flight
        // together), lane 0 sets the barriers up and requests the first pages into the stages (which start empty: no wait).
        const int ahead = min(n, STAGES);
        const int myblock = lane < ahead ? p.block_table[size_t(b) * p.table_stride + pg0 + lane] : 0;
        if (lane == 0) {
            for (int s = 0; s < STAGES; s++) {
                mbar_init(&full[s], 1);
                mbar_init(&empty[s], NWORK);
            }
            mbar_init(&patched, 1);
            s_failed = 0;
            s_issued = 0;
            fence_barrier_init();
        }
        __syncwarp();
#pragma unroll
        for (int s = 0; s < STAGES; s++) {
            const int blk = __shfl_sync(0xffffffffu, myblock, s);
            if (lane == 0 && s < n && issuing) {
                issuing = issue(s, blk);
                next = s + 1;
            }
        }
    }
    if (p.ctl.early) {
        pdl_wait();
        pdl_launch_dependents();
    }
    trace_first(p.ctl.trace, 1);
    // Heads of this kv head into shared memory as fp16 (and fp32 for the scoring chain): optional
    // head norm with gains in the oracle's operation order, rounded to the activation dtype.
    for (int hh = warp; hh < 8; hh += NWORK + 1) {
        float x[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (hh < p.G) {
            const size_t off = size_t(b) * p.q_stride + size_t(kvh * p.G + hh) * HD;
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
            qh[hh][lane + 32 * i] = __float2half_rn(x[i]);
            if (SCORES) qf[hh][lane + 32 * i] = x[i];
        }
    }
    __syncthreads();

    // Lane (g, c) of a consumer warp. S^T = K Q^T: M rows are 16 keys, N columns the 8 (padded)
    // query heads; O^T = V^T P^T: M rows are 16 head dims, K the same 16 keys.
    const int g = lane >> 2, c = lane & 3;
    float OT[8][4];
#pragma unroll
    for (int i = 0; i < 8; i++) OT[i][0] = OT[i][1] = OT[i][2] = OT[i][3] = 0.0f;
    float ps0 = 0.0f, ps1 = 0.0f;   // sums of weights of heads 2c, 2c + 1

    if (warp == NWORK) {
        // ---- producer, after the first pages
        int code[2][4];
        float rscale[2] = {0.0f, 0.0f};
        const int row = (S - 1) & (BLK - 1);
        if (appends) {
            // the whole warp, while the first pages are in flight
            const int block = p.block_table[size_t(b) * p.table_stride + npages - 1];
            uint8_t* page = const_cast<uint8_t*>(p.pool) + ((size_t(block) * p.n_layers + p.layer) * p.n_kv_heads + kvh) * p.page_bytes;
#pragma unroll
            for (int side = 0; side < 2; side++) {
                float x[4];
                kv_row_load<DT>(side ? p.v_new : p.k_new, size_t(b) * p.kv_stride + size_t(kvh) * HD, side == 0 && p.norm_k != 0, lane, x);
                kv_row_quantise<DT>(x, code[side], rscale[side]);
                int8_t* codes = reinterpret_cast<int8_t*>(page) + side * CODE_BYTES + row * HD;
#pragma unroll
                for (int i = 0; i < 4; i++) codes[lane + 32 * i] = int8_t(code[side][i]);
                if (lane == 0) {
                    uint8_t* sc = page + 2 * CODE_BYTES + side * BLK * SB;
                    if (SB == 4) reinterpret_cast<float*>(sc)[row] = rscale[side];
                    else reinterpret_cast<__half*>(sc)[row] = __float2half_rn(rscale[side]);
                }
            }
        }
        if (lane == 0)
            for (; next < n && issuing; next++) issuing = issue(next, -1);
        if (appends) {
            __syncwarp();
            const int il = n - 1;
            uint8_t* Kb = stages + (il % STAGES) * FD_STAGE_BYTES;
            if (mbar_wait_bounded(p.ctl.wait_cycles, &full[il % STAGES], (il / STAGES) & 1)) {
#pragma unroll
                for (int side = 0; side < 2; side++) {
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const int d = lane + 32 * i;
                        Kb[side * CODE_BYTES + row * 128 + (((d >> 4) ^ (row & 7)) << 4) + (d & 15)] = uint8_t(int8_t(code[side][i]));
                    }
                    if (lane == 0) {
                        uint8_t* sc = Kb + 2 * CODE_BYTES + side * BLK * SB;
                        if (SB == 4) reinterpret_cast<float*>(sc)[row] = rscale[side];
                        else reinterpret_cast<__half*>(sc)[row] = __float2half_rn(rscale[side]);
                    }
                }
            } else if (lane == 0) {
                atomicExch(p.ctl.err, ERR_WAIT_FULL);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&patched);
        }
    } else if (SCORES && warp >= NCONS) {
        // ---- scoring warps
        for (int i = 0; i < n; i++) {
            const int st = i % STAGES, use = i / STAGES;
            // (the decision is the warp's: a warp that leaves the loop leaves it whole)
            if (!__all_sync(0xffffffffu, mbar_wait_bounded(p.ctl.wait_cycles, &full[st], use & 1) &&
                                             (!(appends && i == n - 1) || mbar_wait_bounded(p.ctl.wait_cycles, &patched, 0)))) {
                atomicExch(p.ctl.err, ERR_WAIT_FULL);
                *reinterpret_cast<volatile int*>(&s_failed) = 1;
                break;
            }
            const uint8_t* Kb = stages + st * FD_STAGE_BYTES;
            const uint8_t* ksc = Kb + 2 * CODE_BYTES;
            const int key_base = (pg0 + i) * BLK;
            if (SCORES) {
                // One key a thread: the dots of the kv head's heads, each ONE fp32 fma chain over d ascending
                // (the order the CPU restatement fixes; the selection that follows compares index sets bit for bit).
                const int r = (warp - NCONS) * 32 + lane;
                if (key_base + r < S) {
                    float dot[GT > 0 ? GT : 1];
#pragma unroll
                    for (int h = 0; h < GT; h++) dot[h] = 0.0f;
                    const uint8_t* krow = Kb + r * 128;
#pragma unroll
                    for (int ch = 0; ch < 8; ch++) {
                        const uint4 w4 = *reinterpret_cast<const uint4*>(krow + ((ch ^ (r & 7)) << 4));
                        const uint32_t w[4] = {w4.x ^ 0x80808080u, w4.y ^ 0x80808080u, w4.z ^ 0x80808080u, w4.w ^ 0x80808080u};
                        if (DT == EMBLA_F16) {
                            // codes widened exactly to fp16 pairs, queries as stored: the mixed-precision fma multiplies
                            // exactly and rounds each step once to fp32, as fmaf on the converted values would
#pragma unroll
                            for (int h8 = 0; h8 < 2; h8++) {
                                const uint32_t k01 = h2_from_biased_bytes(w[2 * h8], 0x4140), k23 = h2_from_biased_bytes(w[2 * h8], 0x4342);
                                const uint32_t k45 = h2_from_biased_bytes(w[2 * h8 + 1], 0x4140), k67 = h2_from_biased_bytes(w[2 * h8 + 1], 0x4342);
                                const int d = ch * 16 + h8 * 8;
#pragma unroll
                                for (int h = 0; h < GT; h++) {
                                    if (SG != 9 || h < p.G) {
                                        const uint4 q8 = *reinterpret_cast<const uint4*>(&qh[h][d]);   // one address a warp
                                        fma_pair_f16(dot[h], k01, q8.x);
                                        fma_pair_f16(dot[h], k23, q8.y);
                                        fma_pair_f16(dot[h], k45, q8.z);
                                        fma_pair_f16(dot[h], k67, q8.w);
                                    }
                                }
                            }
                        } else {
#pragma unroll
                            for (int e4 = 0; e4 < 4; e4++) {
                                const float k0 = f32_from_biased_byte(w[e4], 0), k1 = f32_from_biased_byte(w[e4], 1);
                                const float k2 = f32_from_biased_byte(w[e4], 2), k3 = f32_from_biased_byte(w[e4], 3);
                                const int d = ch * 16 + e4 * 4;
#pragma unroll
                                for (int h = 0; h < GT; h++) {
                                    if (SG != 9 || h < p.G) {
                                        const float4 q4 = *reinterpret_cast<const float4*>(&qf[h][d]);
                                        dot[h] = __fmaf_rn(q4.x, k0, dot[h]);
                                        dot[h] = __fmaf_rn(q4.y, k1, dot[h]);
                                        dot[h] = __fmaf_rn(q4.z, k2, dot[h]);
                                        dot[h] = __fmaf_rn(q4.w, k3, dot[h]);
                                    }
                                }
                            }
                        }
                    }
                    const float ks = ld_scale<SB>(ksc, r);
                    float best = __fmul_rn(dot[0], ks);
#pragma unroll
                    for (int h = 1; h < GT; h++) {
                        if (SG != 9 || h < p.G) {
                            const float t = __fmul_rn(dot[h], ks);
                            if (t > best) best = t;
                        }
                    }
                    p.scores[(size_t(b) * p.n_kv_heads + kvh) * p.scores_stride + key_base + r] = best;
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[st]);
        }
    } else {
        // ---- consumers
        uint32_t qb0[8], qb1[8];
#pragma unroll
        for (int t = 0; t < 8; t++) {
            const int d0 = (t < 4) ? 16 * c + 4 * t : 64 + 16 * c + 4 * (t - 4);
            qb0[t] = *reinterpret_cast<const uint32_t*>(&qh[g][d0]);
            qb1[t] = *reinterpret_cast<const uint32_t*>(&qh[g][d0 + 2]);
        }
        const int rg = rho(g), kA = rho(2 * c), kB = kA ^ 4;
        const float scale = rsqrtf(float(HD));
        for (int i = 0; i < n; i++) {
            const int st = i % STAGES, use = i / STAGES;
            // (the decision is the warp's: a warp that leaves the loop leaves it whole)
            if (!__all_sync(0xffffffffu, mbar_wait_bounded(p.ctl.wait_cycles, &full[st], use & 1) &&
                                             (!(appends && i == n - 1) || mbar_wait_bounded(p.ctl.wait_cycles, &patched, 0)))) {
                atomicExch(p.ctl.err, ERR_WAIT_FULL);
                *reinterpret_cast<volatile int*>(&s_failed) = 1;
                break;
            }
            const uint8_t* Kb = stages + st * FD_STAGE_BYTES;
            const uint8_t* Vb = Kb + CODE_BYTES;
            const uint8_t* ksc = Kb + 2 * CODE_BYTES;
            const uint8_t* vsc = ksc + BLK * SB;
            const int key_base = (pg0 + i) * BLK;

#pragma unroll
            for (int step = 0; step < KPW / 16; step++) {
                const int R0 = warp * KPW + step * 16;
                const int r0 = R0 + rg, r1 = r0 + 8;
                float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                {
                    const uint8_t* k0 = Kb + r0 * 128;
                    const uint4 lo0 = *reinterpret_cast<const uint4*>(k0 + ((c ^ rg) << 4));
                    const uint4 hi0 = *reinterpret_cast<const uint4*>(k0 + (((c + 4) ^ rg) << 4));
                    const uint4 lo1 = *reinterpret_cast<const uint4*>(k0 + 8 * 128 + ((c ^ rg) << 4));
                    const uint4 hi1 = *reinterpret_cast<const uint4*>(k0 + 8 * 128 + (((c + 4) ^ rg) << 4));
                    const uint32_t w0[8] = {lo0.x, lo0.y, lo0.z, lo0.w, hi0.x, hi0.y, hi0.z, hi0.w};
                    const uint32_t w1[8] = {lo1.x, lo1.y, lo1.z, lo1.w, hi1.x, hi1.y, hi1.z, hi1.w};
#pragma unroll
                    for (int t = 0; t < 8; t++) {
                        const uint32_t x0 = w0[t] ^ 0x80808080u, x1 = w1[t] ^ 0x80808080u;
                        mma_16816(s, h2_from_biased_bytes(x0, 0x4140), h2_from_biased_bytes(x1, 0x4140),
                                  h2_from_biased_bytes(x0, 0x4342), h2_from_biased_bytes(x1, 0x4342), qb0[t], qb1[t]);
                    }
                }
                // s[0], s[1]: key r0, heads 2c, 2c+1; s[2], s[3]: key r1
                const bool v0 = key_base + r0 < S, v1 = key_base + r1 < S;
                const float ks0 = ld_scale<SB>(ksc, r0), ks1 = ld_scale<SB>(ksc, r1);
                const float a00 = fmaxf(s[0] * ks0 * scale, 0.0f), a01 = fmaxf(s[1] * ks0 * scale, 0.0f);
                const float a10 = fmaxf(s[2] * ks1 * scale, 0.0f), a11 = fmaxf(s[3] * ks1 * scale, 0.0f);
                const float w00 = v0 ? a00 * a00 : 0.0f, w01 = v0 ? a01 * a01 : 0.0f;
                const float w10 = v1 ? a10 * a10 : 0.0f, w11 = v1 ? a11 * a11 : 0.0f;
                ps0 += w00 + w10;
                ps1 += w01 + w11;
                // V-skip: a 16-key tile whose weights are all zero adds nothing (attention.metal:310)
                const bool live = (w00 != 0.0f) | (w01 != 0.0f) | (w10 != 0.0f) | (w11 != 0.0f);
                if (!__any_sync(0xffffffffu, live)) continue;
                const float vs0 = v0 ? ld_scale<SB>(vsc, r0) : 0.0f, vs1 = v1 ? ld_scale<SB>(vsc, r1) : 0.0f;
                const uint32_t pb0 = movmatrix_trans(pack_h2(w00 * vs0, w01 * vs0));
                const uint32_t pb1 = movmatrix_trans(pack_h2(w10 * vs1, w11 * vs1));
                const uint8_t* vA = Vb + (R0 + kA) * 128 + ((g ^ kA) << 4);
                const uint8_t* vB = Vb + (R0 + kB) * 128 + ((g ^ kB) << 4);
                const uint4 a4 = *reinterpret_cast<const uint4*>(vA);
                const uint4 b4 = *reinterpret_cast<const uint4*>(vB);
                const uint4 c4 = *reinterpret_cast<const uint4*>(vA + 8 * 128);
                const uint4 d4 = *reinterpret_cast<const uint4*>(vB + 8 * 128);
                const uint32_t va[4] = {a4.x, a4.y, a4.z, a4.w}, vb[4] = {b4.x, b4.y, b4.z, b4.w};
                const uint32_t vc[4] = {c4.x, c4.y, c4.z, c4.w}, vd[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
                for (int wq = 0; wq < 2; wq++) {
                    // dims 16g + 4wq + e (rows g of tiles 4wq + e) and 16g + 8 + 4wq + e (rows g + 8)
                    const uint32_t xl = va[wq] ^ 0x80808080u, yl = vb[wq] ^ 0x80808080u;
                    const uint32_t xh = va[wq + 2] ^ 0x80808080u, yh = vb[wq + 2] ^ 0x80808080u;
                    const uint32_t x2l = vc[wq] ^ 0x80808080u, y2l = vd[wq] ^ 0x80808080u;
                    const uint32_t x2h = vc[wq + 2] ^ 0x80808080u, y2h = vd[wq + 2] ^ 0x80808080u;
                    const uint32_t zl0 = __byte_perm(xl, yl, 0x5140), zl1 = __byte_perm(xl, yl, 0x7362);
                    const uint32_t zh0 = __byte_perm(xh, yh, 0x5140), zh1 = __byte_perm(xh, yh, 0x7362);
                    const uint32_t ul0 = __byte_perm(x2l, y2l, 0x5140), ul1 = __byte_perm(x2l, y2l, 0x7362);
                    const uint32_t uh0 = __byte_perm(x2h, y2h, 0x5140), uh1 = __byte_perm(x2h, y2h, 0x7362);
                    mma_16816(OT[4 * wq + 0], h2_from_biased_bytes(zl0, 0x4140), h2_from_biased_bytes(zh0, 0x4140),
                              h2_from_biased_bytes(ul0, 0x4140), h2_from_biased_bytes(uh0, 0x4140), pb0, pb1);
                    mma_16816(OT[4 * wq + 1], h2_from_biased_bytes(zl0, 0x4342), h2_from_biased_bytes(zh0, 0x4342),
                              h2_from_biased_bytes(ul0, 0x4342), h2_from_biased_bytes(uh0, 0x4342), pb0, pb1);
                    mma_16816(OT[4 * wq + 2], h2_from_biased_bytes(zl1, 0x4140), h2_from_biased_bytes(zh1, 0x4140),
                              h2_from_biased_bytes(ul1, 0x4140), h2_from_biased_bytes(uh1, 0x4140), pb0, pb1);
                    mma_16816(OT[4 * wq + 3], h2_from_biased_bytes(zl1, 0x4342), h2_from_biased_bytes(zh1, 0x4342),
                              h2_from_biased_bytes(ul1, 0x4342), h2_from_biased_bytes(uh1, 0x4342), pb0, pb1);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[st]);
        }
    }

    trace_last(p.ctl.trace, 2);
    // ---- the consumer warps' sums into one partial. The stage ring is free now: every page that
    // was requested has been waited for, unless a wait gave up — then wait (bounded) for what is
    // still in flight first.
    __syncthreads();
    if (s_failed) {
        if (tid == 0) {
            for (int i = max(0, s_issued - STAGES); i < s_issued; i++)
                if (!mbar_wait_bounded(p.ctl.wait_cycles, &full[i % STAGES], (i / STAGES) & 1)) atomicExch(p.ctl.err, ERR_WAIT_DRAIN);
        }
        __syncthreads();
    }
    float(*red)[8][HD] = reinterpret_cast<float(*)[8][HD]>(stages);
    float(*redp)[8] = reinterpret_cast<float(*)[8]>(stages + NCONS * 8 * HD * 4);
    if (warp < NCONS) {
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
            ps0 += __shfl_xor_sync(0xffffffffu, ps0, o);
            ps1 += __shfl_xor_sync(0xffffffffu, ps1, o);
        }
#pragma unroll
        for (int i = 0; i < 8; i++) {
            red[warp][2 * c][16 * g + i] = OT[i][0];
            red[warp][2 * c + 1][16 * g + i] = OT[i][1];
            red[warp][2 * c][16 * g + 8 + i] = OT[i][2];
            red[warp][2 * c + 1][16 * g + 8 + i] = OT[i][3];
        }
        if (g == 0) {
            redp[warp][2 * c] = ps0;
            redp[warp][2 * c + 1] = ps1;
        }
    }
    __syncthreads();

    const int pair = b * p.n_kv_heads + kvh;
    const float sink = sqrtf(float(HD));
    float* part = p.partials + (size_t(pair) * p.nsplit + split) * p.G * FD_PART;
    // (clusters) rows [sender][head of this owner] that the other ranges write into this CTA's shared memory
    float* inbox = reinterpret_cast<float*>(smem + fd_inbox_offset(STAGES, SCORES));
    const int slots = CL ? (p.G + p.nsplit - 1) / p.nsplit : 0;   // heads an owner finishes
    for (int idx = tid; idx < p.G * HD; idx += THREADS) {
        const int hh = idx >> 7, d = idx & 127;
        float num = 0.0f, den = 0.0f;
#pragma unroll
        for (int w = 0; w < NCONS; w++) {
            num += red[w][hh][d];
            den += redp[w][hh];
        }
        if (p.nsplit == 1) {
            Act<DT>::store(p.o, size_t(b) * p.o_stride + size_t(kvh * p.G + hh) * HD + d, num / (sink + den));
        } else if (CL) {
            const uint32_t row = cluster_map(smem_u32(inbox + (split * slots + hh / p.nsplit) * FD_PART), uint32_t(hh % p.nsplit));
            cluster_st_f32(row + uint32_t(d) * 4u, num);
            if (d == 0) cluster_st_f32(row + HD * 4, den);
        } else {
            part[hh * FD_PART + d] = num;
            if (d == 0) part[hh * FD_PART + HD] = den;
        }
    }
    if (CL && p.nsplit > 1) {
        // one cluster barrier: every range's rows are in their owners' inboxes; CTA `split` adds the rows of heads
        // split, split + nsplit, ... in range order from its own shared memory and is done
        cluster_arrive();
        cluster_wait();
        for (int idx = tid; idx < slots * HD; idx += THREADS) {
            const int slot = idx >> 7, d = idx & 127, hh = split + slot * p.nsplit;
            if (hh < p.G) {
                float num = 0.0f, den = sink;
                for (int r = 0; r < p.nsplit; r++) {
                    const float* row = inbox + (r * slots + slot) * FD_PART;
                    den += row[HD];
                    num += row[d];
                }
                Act<DT>::store(p.o, size_t(b) * p.o_stride + size_t(kvh * p.G + hh) * HD + d, num / den);
            }
        }
        trace_last(p.ctl.trace, 3);
        return;
    }
    if (p.nsplit == 1) {
        trace_last(p.ctl.trace, 3);
        return;
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
    if (!s_last) {
        trace_last(p.ctl.trace, 3);
        return;
    }
    __threadfence();
    const float* base = p.partials + size_t(pair) * p.nsplit * p.G * FD_PART;
    const int n4 = p.nsplit * p.G * (FD_PART / 4);
    if (n4 * 16 <= STAGES * FD_STAGE_BYTES) {
        // the pair's partials (contiguous: [split][head][128 sums, sum of weights]) into the free stages in one batch of
        // loads, then added in split order from shared memory
        float* sbase = reinterpret_cast<float*>(stages);
        stage_from_global<THREADS>(reinterpret_cast<float4*>(sbase), reinterpret_cast<const float4*>(base), n4, tid);
        __syncthreads();
        for (int idx = tid; idx < p.G * HD; idx += THREADS) {
            const int hh = idx >> 7, d = idx & 127;
            float num = 0.0f, den = sink;
            for (int s = 0; s < p.nsplit; s++) {
                const float* q2 = sbase + (s * p.G + hh) * FD_PART;
                den += q2[HD];
                num += q2[d];
            }
            Act<DT>::store(p.o, size_t(b) * p.o_stride + size_t(kvh * p.G + hh) * HD + d, num / den);
        }
    } else {
        for (int idx = tid; idx < p.G * HD; idx += THREADS) {
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
    trace_last(p.ctl.trace, 3);
}

template <int STAGES, bool SCORES>
constexpr size_t fd_smem_bytes() {
    return 1024 + size_t(STAGES) * FD_STAGE_BYTES + 8 * HD * 2 + 2 * STAGES * 8 + (SCORES ? 8 * QF_LD * 4 : 0);
}
// Cluster launches (at most 4 ranges) add the inbox: ranges x ceil(heads / ranges) rows of FD_PART floats, at most 6 rows
// for up to 4 query heads a kv head, 9 for 8.
constexpr int fd_inbox_rows(int G) { return G <= 4 ? 6 : 9; }

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

// The split of the attention-only (no scores) launch: up to 4 ranges a pair may run as one thread-block cluster that
// combines through its shared memory, which saves the round trip through global scratch (worth about a page of
// streaming); larger clusters leave SMs of a GPC idle, so more ranges than that combine through the scratch. The split is a
// function of the shape only: every entry point that runs this kernel cuts a pair the same way and so adds in the same order.
int choose_full_decode_split(int pairs, int pages, int slots, int max_slots, bool* cluster) {
    const int any = choose_splits(pairs, pages, slots, max_slots);
    const int few = choose_splits(pairs, pages, slots, 4 * pairs);
    auto cost = [&](int ns) {
        const long waves = (long(pairs) * ns + slots - 1) / slots;
        return double(waves) * ((pages + ns - 1) / ns + 3.0);
    };
    static const bool use_clusters = []() { const char* e = getenv("EMBLA_NO_CLUSTER"); return !(e && e[0] == '1'); }();
    if (use_clusters && few > 1 && cost(few) <= cost(any) + 1.0) {
        *cluster = true;
        return few;
    }
    *cluster = false;
    return any;
}

}  // namespace embla

using namespace embla;

template <int DT, int SB, int SG, bool CL>
static EmblaStatus launch_full_decode_cl(EmblaAttn* ctx, const EmblaKVPool* pool, const FullDecodeParams& p, int batch,
                                         cudaStream_t s) {
    constexpr int STAGES = 3;
    constexpr bool SCORES = SG != 0;
    constexpr int NCONS = SCORES ? 4 : 8;
    constexpr int FD_THREADS = (NCONS + (SCORES ? 4 : 0) + 1) * 32;
    const size_t smem = CL ? 1024 + fd_inbox_offset(STAGES, SCORES) + size_t(fd_inbox_rows(p.G)) * FD_PART * 4 : fd_smem_bytes<STAGES, SCORES>();
    auto kern = full_decode_kernel<DT, SB, NCONS, STAGES, SG, CL>;
    static bool configured[64] = {};   // per instantiation and device
    if (!configured[ctx->device & 63]) {
        EMBLA_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            int(CL ? 1024 + fd_inbox_offset(STAGES, SCORES) + 9 * FD_PART * 4 : fd_smem_bytes<STAGES, SCORES>())));
        configured[ctx->device & 63] = true;
    }
    dim3 grid(p.nsplit, p.n_kv_heads, batch);
    EMBLA_CUDA_TRY(launch_kernel_cluster(ctx->pdl, CL ? p.nsplit : 1, kern, grid, dim3(FD_THREADS), smem, s, pool->tmap_codes, p));
    EMBLA_CUDA_TRY(cudaGetLastError());
    return EMBLA_OK;
}

template <int DT, int SB, int SG>
static EmblaStatus launch_full_decode(EmblaAttn* ctx, const EmblaKVPool* pool, const FullDecodeParams& p, int batch,
                                      bool cluster, cudaStream_t s) {
    // (the scoring variant keeps the combine through global scratch: with its fp32 queries the inbox would not leave room
    // for two CTAs an SM)
    if (SG == 0 && cluster) return launch_full_decode_cl<DT, SB, SG, SG == 0>(ctx, pool, p, batch, s);
    return launch_full_decode_cl<DT, SB, SG, false>(ctx, pool, p, batch, s);
}

static EmblaStatus full_decode_impl(EmblaAttn* ctx, const EmblaKVPool* pool, const EmblaKVView* view, const EmblaQuery* q,
                                    void* o_dev, int64_t o_stride, float* scores_dev, int64_t scores_stride, const void* k_new,
                                    const void* v_new, int64_t kv_stride, int32_t norm_k, void* stream) {
    if (!ctx || !pool || !view || !q || !o_dev) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_full_decode: null argument");
    EMBLA_CHECK_DEVICE("embla_attn_full_decode", ctx, pool);
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

    if (pool->kv_dtype == EMBLA_KV_16BIT) {
        // The reference's build without the int8 cache (EMBLA_KV8=0: attn_full, attention.metal:148-220): the rows are stored
        // in the activation dtype and the same entry point serves it, as separate launches: the key scores (SCORES: the
        // scoring pass of the sparse layers, which needs the queries as they enter the dot products), then the ReLU²
        // attention over every key. The token's row is appended with embla_kv_append beforehand.
        if (k_new) {
            EMBLA_FAIL(EMBLA_UNSUPPORTED, "embla_attn_full_step: a 16-bit pool takes embla_kv_append, then embla_attn_full_decode");
        }
        if (scores_dev) {
            if (!q->prenormed) EMBLA_FAIL(EMBLA_UNSUPPORTED, "embla_attn_full_decode: key scores over a 16-bit pool need prenormed queries");
            if (EmblaStatus st = embla_score_keys(ctx, pool, view, q->q_dev, q->q_stride, scores_dev, scores_stride, stream)) return st;
        }
        return attn16_full_decode(ctx, pool, view, q, o_dev, o_stride, max_len, static_cast<cudaStream_t>(stream));
    }
    if (pool->kv_dtype != EMBLA_KV_INT8) EMBLA_FAIL(EMBLA_UNSUPPORTED, "embla_attn_full_decode: unknown pool dtype %d", pool->kv_dtype);

    FullDecodeParams p = {};
    p.pool = pool->base;
    p.block_table = view->block_table_dev;
    p.seq_lens = view->seq_lens_dev;
    p.q = q->q_dev;
    p.g1 = q->g1_dev;
    p.g2 = q->g2_dev;
    p.o = o_dev;
    p.partials = ctx->partials;
    p.counters = ctx->counters;
    p.ctl = kernel_ctl(ctx);
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
    p.k_new = k_new;
    p.v_new = v_new;
    p.kv_stride = kv_stride;
    p.norm_k = norm_k;
    const int pairs = view->batch * pool->n_kv_heads;
    const int pages = (max_len + BLK - 1) / BLK;
    bool cluster = false;
    if (scores_dev) p.nsplit = choose_splits(pairs, pages, 2 * ctx->sm_count, ctx->partial_slots);
    else p.nsplit = choose_full_decode_split(pairs, pages, 2 * ctx->sm_count, ctx->partial_slots, &cluster);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool bf = ctx->cfg.act_dtype == EMBLA_BF16;
    const bool s4 = pool->scale_bytes == 4;
#define EMBLA_FD(DT, SB, SC) launch_full_decode<DT, SB, SC>(ctx, pool, p, view->batch, cluster, s)
#define EMBLA_FD_SG(SG) \
    (bf ? (s4 ? EMBLA_FD(EMBLA_BF16, 4, SG) : EMBLA_FD(EMBLA_BF16, 2, SG)) : (s4 ? EMBLA_FD(EMBLA_F16, 4, SG) : EMBLA_FD(EMBLA_F16, 2, SG)))
    if (scores_dev) {   // the head count compiled in for the usual groupings
        switch (p.G) {
            case 1: return EMBLA_FD_SG(1);
            case 2: return EMBLA_FD_SG(2);
            case 4: return EMBLA_FD_SG(4);
            case 8: return EMBLA_FD_SG(8);
            default: return EMBLA_FD_SG(9);
        }
    }
    return EMBLA_FD_SG(0);
#undef EMBLA_FD_SG
#undef EMBLA_FD
}

extern "C" EmblaStatus embla_attn_full_decode(EmblaAttn* ctx, const EmblaKVPool* pool, const EmblaKVView* view,
                                              const EmblaQuery* q, void* o_dev, int64_t o_stride,
                                              float* scores_dev, int64_t scores_stride, void* stream) {
    return full_decode_impl(ctx, pool, view, q, o_dev, o_stride, scores_dev, scores_stride, nullptr, nullptr, 0, 0, stream);
}

extern "C" EmblaStatus embla_attn_full_step(EmblaAttn* ctx, EmblaKVPool* pool, const EmblaKVView* view, const EmblaQuery* q,
                                            const void* k_dev, const void* v_dev, int64_t kv_stride, int32_t norm_k,
                                            void* o_dev, int64_t o_stride, float* scores_dev, int64_t scores_stride,
                                            void* stream) {
    if (!k_dev || !v_dev) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_full_step: null k or v");
    return full_decode_impl(ctx, pool, view, q, o_dev, o_stride, scores_dev, scores_stride, k_dev, v_dev, kv_stride, norm_k, stream);
}

// ---- full-layer decode for callers that must not allocate ---------------------------------------------
// Some hosts of this library cannot call cudaMalloc at the point where they run attention: a serving
// loop that has handed all device memory to its own arena at start-up, or a latency-critical thread
// in which an allocation (and the device-wide synchronisation it can imply) is forbidden. For them
// this entry point runs the same kernel as embla_attn_full_decode without any context object: the
// split-K partial sums, the arrival counters and the error word live in the fixed array below, which
// every GPU that loads the library holds from load to exit.
namespace embla {

constexpr int NOALLOC_MAX_PAIRS = 256;     // batch x kv heads
constexpr int NOALLOC_MAX_SLOTS = 1024;    // (pair, key range) partials
constexpr size_t NOALLOC_COUNTER_BYTES = NOALLOC_MAX_PAIRS * sizeof(int);          // 1 KiB
constexpr size_t NOALLOC_ERR_OFFSET = NOALLOC_COUNTER_BYTES;                        // one int, own 256-byte line
constexpr size_t NOALLOC_PART_OFFSET = NOALLOC_COUNTER_BYTES + 256;
constexpr size_t NOALLOC_BYTES = NOALLOC_PART_OFFSET + size_t(NOALLOC_MAX_SLOTS) * 8 * FD_PART * sizeof(float);   // ~4.1 MiB

// In host code this name is only a handle for the runtime, not a device address: the address the
// kernel gets comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_BYTES];

struct NoAllocDevice {
    bool ready;
    unsigned char* scratch;
    int sm_count;
};
static NoAllocDevice g_noalloc[64];

// Once per device, with that device current: resolve the array's device address and let the kernel
// variants use their dynamic shared memory. Nothing here allocates.
template <int DT, int SB>
static EmblaStatus noalloc_setup_kernel() {
    constexpr size_t smem = fd_smem_bytes<3, false>();
    EMBLA_CUDA_TRY(cudaFuncSetAttribute(full_decode_kernel<DT, SB, 8, 3, 0, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        int(smem)));
    return EMBLA_OK;
}

static EmblaStatus noalloc_setup(int device) {
    NoAllocDevice& d = g_noalloc[device];
    if (d.ready) return EMBLA_OK;
    void* ptr = nullptr;
    EMBLA_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
    EMBLA_CUDA_TRY(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, device));
    if (EmblaStatus s = noalloc_setup_kernel<EMBLA_BF16, 4>()) return s;
    if (EmblaStatus s = noalloc_setup_kernel<EMBLA_BF16, 2>()) return s;
    if (EmblaStatus s = noalloc_setup_kernel<EMBLA_F16, 4>()) return s;
    if (EmblaStatus s = noalloc_setup_kernel<EMBLA_F16, 2>()) return s;
    d.scratch = static_cast<unsigned char*>(ptr);
    d.ready = true;
    return EMBLA_OK;
}

}  // namespace embla

extern "C" EmblaStatus embla_attn_full_decode_noalloc(const EmblaKVPool* pool, const EmblaKVView* view, const EmblaQuery* q,
                                                      int32_t n_q_heads, int32_t act_dtype, void* o_dev, int64_t o_stride,
                                                      void* stream) {
    if (!pool || !view || !q || !o_dev) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_full_decode_noalloc: null argument");
    if (pool->kv_dtype != EMBLA_KV_INT8) EMBLA_FAIL(EMBLA_UNSUPPORTED, "embla_attn_full_decode_noalloc: the pool is not int8");
    if (act_dtype != EMBLA_BF16 && act_dtype != EMBLA_F16)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_full_decode_noalloc: act_dtype %d", act_dtype);
    const int Hkv = pool->n_kv_heads;
    if (n_q_heads <= 0 || n_q_heads % Hkv != 0 || n_q_heads / Hkv > 8)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_full_decode_noalloc: %d query heads on %d kv heads", n_q_heads, Hkv);
    if (view->layer < 0 || view->layer >= pool->n_layers || !view->block_table_dev || !view->seq_lens_dev || !q->q_dev)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_full_decode_noalloc: bad view or query");
    if (!q->prenormed && ((q->ng >= 1 && !q->g1_dev) || (q->ng >= 2 && !q->g2_dev) || q->ng < 0 || q->ng > 2))
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_full_decode_noalloc: ng %d without its gain vectors", q->ng);
    if (view->batch <= 0 || long(view->batch) * Hkv > NOALLOC_MAX_PAIRS)
        EMBLA_FAIL(EMBLA_BAD_ARG,
                   "embla_attn_full_decode_noalloc: batch %d x %d kv heads is over the fixed scratch's limit of %d "
                   "(sequence, kv head) pairs; use embla_attn_full_decode with a context sized for it",
                   view->batch, Hkv, NOALLOC_MAX_PAIRS);
    if (view->max_seq_len <= 0)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_full_decode_noalloc: max_seq_len must be given (there is no context to take it from)");
    int device = 0;
    EMBLA_CUDA_TRY(cudaGetDevice(&device));
    if (device < 0 || device >= 64) EMBLA_FAIL(EMBLA_UNSUPPORTED, "embla_attn_full_decode_noalloc: device %d", device);
    if (device != pool->device) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_full_decode_noalloc: the pool lives on device %d", pool->device);
    if (EmblaStatus s = noalloc_setup(device)) return s;
    const NoAllocDevice& d = g_noalloc[device];
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // The array keeps what the last call left: counters and the error word must start at zero.
    EMBLA_CUDA_TRY(cudaMemsetAsync(d.scratch, 0, NOALLOC_PART_OFFSET, s));

    FullDecodeParams p = {};
    p.pool = pool->base;
    p.block_table = view->block_table_dev;
    p.seq_lens = view->seq_lens_dev;
    p.q = q->q_dev;
    p.g1 = q->g1_dev;
    p.g2 = q->g2_dev;
    p.o = o_dev;
    p.counters = reinterpret_cast<int*>(d.scratch);
    p.ctl.err = reinterpret_cast<int*>(d.scratch + NOALLOC_ERR_OFFSET);
    p.ctl.trace = nullptr;
    p.ctl.wait_cycles = WAIT_CYCLES;
    p.ctl.stall_at = -1;
    p.ctl.early = 0;
    p.partials = reinterpret_cast<float*>(d.scratch + NOALLOC_PART_OFFSET);
    p.scores = nullptr;
    p.q_stride = q->q_stride;
    p.o_stride = o_stride;
    p.scores_stride = 0;
    p.page_bytes = pool->page_bytes;
    p.table_stride = view->table_stride;
    p.layer = view->layer;
    p.n_layers = pool->n_layers;
    p.n_kv_heads = Hkv;
    p.G = n_q_heads / Hkv;
    p.scale_bytes = pool->scale_bytes;
    p.rows_per_page = pool->rows_per_page;
    p.prenormed = q->prenormed;
    p.ng = q->ng;
    const int pairs = view->batch * Hkv;
    const int pages = (view->max_seq_len + BLK - 1) / BLK;
    bool cluster_unused = false;   // (this entry point always combines through its fixed scratch)
    p.nsplit = choose_full_decode_split(pairs, pages, 2 * d.sm_count, NOALLOC_MAX_SLOTS, &cluster_unused);
    constexpr size_t smem = fd_smem_bytes<3, false>();
    dim3 grid(p.nsplit, Hkv, view->batch);
    const bool s4 = pool->scale_bytes == 4;
    if (act_dtype == EMBLA_BF16) {
        if (s4) full_decode_kernel<EMBLA_BF16, 4, 8, 3, 0, false><<<grid, 9 * 32, smem, s>>>(pool->tmap_codes, p);
        else full_decode_kernel<EMBLA_BF16, 2, 8, 3, 0, false><<<grid, 9 * 32, smem, s>>>(pool->tmap_codes, p);
    } else {
        if (s4) full_decode_kernel<EMBLA_F16, 4, 8, 3, 0, false><<<grid, 9 * 32, smem, s>>>(pool->tmap_codes, p);
        else full_decode_kernel<EMBLA_F16, 2, 8, 3, 0, false><<<grid, 9 * 32, smem, s>>>(pool->tmap_codes, p);
    }
    EMBLA_CUDA_TRY(cudaGetLastError());
    return EMBLA_OK;
}
