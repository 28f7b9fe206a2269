// Softmax decode attention over 16-bit keys and values, one query token per sequence:
//  * sparse layers (Sources/EmblaMetal/Kernels/attention.metal:370-441, 448-584, 593-645; dispatch
//    Sources/EmblaMetal/Engine.swift:796-818): every key while the sequence has at most 1152, else
//    the 1152 selected rows idx[kv head][..] gathered from the paged pool;
//  * sliding layers (attention.metal:26-102): the last `window` positions of a ring, after the
//    ring write of the current token (sliding_write_kernel; attention.metal:47-62 and
//    kv_sliding_b, Sources/EmblaMetal/Kernels/prefill.metal:105-125).
//
// One CTA takes 128 rows of one (sequence, kv head): 16-byte cp.async gathers (row address from the
// index list / block table / ring slot) fill swizzled K and V tiles, 4 warps take 32 rows each.
// S^T = K Q^T and O^T = V^T P^T run as m16n8k16 tensor tiles on the 16-bit data as stored; the
// softmax is exact within the CTA (one pass over its rows), and chunks merge through (max, sum,
// acc) partials by the last CTA to arrive, in chunk order (attention.metal:428-440).
#include "attn16_common.cuh"

namespace embla {

constexpr int A16_THREADS = 128;
constexpr int A16_TILE = BLK * HD * 2;      // bytes of a 128-row 16-bit tile
constexpr int A16_PART = HD + 4;            // floats per (chunk, head): 128 sums, max, sum
enum { A16_SPARSE = 0, A16_SLIDING = 1 };

struct Attn16Params {
    const uint8_t* pool;
    const int32_t* block_table;
    const uint32_t* idx;
    const uint8_t* ring_k;
    const uint8_t* ring_v;
    const int32_t* seq_lens;
    const void* q;
    const void* g1;
    const void* g2;
    void* o;
    float* partials;
    int* counters;
    int64_t q_stride, o_stride, ring_stride;   // elements; ring_stride between sequences
    size_t page_bytes;
    int table_stride, layer, n_layers, n_kv_heads, G, prenormed, ng, ring, window, max_chunks;
    // sliding layers, fused ring write of the current token (attention.metal:47-62): its raw k, v rows or NULL
    const void* k_new;
    const void* v_new;
    const void* kgain;
    int64_t kv_stride;
    int k_prenormed;
    float rope_freq[32];
};

template <int DT, int MODE>
__global__ void __launch_bounds__(A16_THREADS) attn16_decode_kernel(const Attn16Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* Kt = smem;                    // [2 halves][128 rows][128 B], chunk ^ (row % 8)
    uint8_t* Vt = smem + A16_TILE;
    uint16_t(*qs)[HD] = reinterpret_cast<uint16_t(*)[HD]>(smem + 2 * A16_TILE);   // [8][128] activation dtype
    __shared__ int s_last;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int chunk = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int S = p.seq_lens[b];
    const bool selecting = MODE == A16_SPARSE && S > EMBLA_TOPK + EMBLA_RECENT;
    const int count = MODE == A16_SLIDING ? min(S, p.window) : (selecting ? EMBLA_TOPK + EMBLA_RECENT : S);
    const int nch = (count + BLK - 1) / BLK;
    if (chunk >= nch) return;
    const int j0 = chunk * BLK;
    const int pos = S - 1;

    // ---- gather this chunk's K and V rows
    {
        const int ch = tid & 15, half = ch >> 3, cc = ch & 7;
#pragma unroll 4
        for (int it = 0; it < 16; it++) {
            const int key = it * 8 + (tid >> 4), j = j0 + key;
            const bool valid = j < count;
            const uint8_t *ksrc, *vsrc;
            if (MODE == A16_SLIDING) {
                const int slot = valid ? (pos - j) % p.ring : 0;
                const size_t off = (size_t(b) * p.ring_stride + (size_t(kvh) * p.ring + slot) * HD) * 2 + ch * 16;
                ksrc = p.ring_k + off;
                vsrc = p.ring_v + off;
            } else {
                int row = valid ? j : 0;
                if (selecting && valid) row = int(p.idx[(size_t(b) * p.n_kv_heads + kvh) * (EMBLA_TOPK + EMBLA_RECENT) + j]);
                const int block = p.block_table[size_t(b) * p.table_stride + (row >> 7)];
                const uint8_t* page = p.pool + ((size_t(block) * p.n_layers + p.layer) * p.n_kv_heads + kvh) * p.page_bytes;
                ksrc = page + (row & 127) * (HD * 2) + ch * 16;
                vsrc = ksrc + A16_TILE;
            }
            const int dst = half * (BLK * 128) + key * 128 + ((cc ^ (key & 7)) << 4);
            cp_async16(Kt + dst, ksrc, valid);
            cp_async16(Vt + dst, vsrc, valid);
        }
    }
    // ---- the kv head's queries (norm, RoPE for sliding layers) while the rows arrive
    for (int hh = warp; hh < 8; hh += A16_THREADS / 32) {
        float x[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (hh < p.G) {
            const size_t off = size_t(b) * p.q_stride + size_t(kvh * p.G + hh) * HD;
#pragma unroll
            for (int i = 0; i < 4; i++) x[i] = Act<DT>::load(p.q, off + lane + 32 * i);
            if (!p.prenormed) norm_rope_round<DT>(x, p.g1, p.g2, p.ng, MODE == A16_SLIDING ? pos : -1, p.rope_freq, lane);
        }
#pragma unroll
        for (int i = 0; i < 4; i++) Act<DT>::store(&qs[hh][0], lane + 32 * i, x[i]);
    }
    cp_async_wait_all();
    if (MODE == A16_SLIDING && p.k_new != nullptr && chunk == 0 && warp == 0) {
        // The current token's key and value (row 0 of this chunk) come from the qkv row, not from the ring: normed,
        // rotated and rounded as attn_sliding does, stored to the ring slot for the steps to come and put in the tiles.
        __syncwarp();
        const size_t off = size_t(b) * p.kv_stride + size_t(kvh) * HD;
        float x[4];
#pragma unroll
        for (int i = 0; i < 4; i++) x[i] = Act<DT>::load(p.k_new, off + lane + 32 * i);
        if (!p.k_prenormed) norm_rope_round<DT>(x, p.kgain, p.kgain, 1, pos, p.rope_freq, lane);
        const size_t slot_off = size_t(b) * p.ring_stride + (size_t(kvh) * p.ring + pos % p.ring) * HD;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int d = lane + 32 * i;
            const int at = (d >> 6) * (BLK * 128) + (((d >> 3) & 7) << 4) + (d & 7) * 2;   // row 0: no swizzle offset
            const uint16_t vbits = reinterpret_cast<const uint16_t*>(p.v_new)[off + d];
            Act<DT>::store(Kt + at, 0, x[i]);
            *reinterpret_cast<uint16_t*>(Vt + at) = vbits;
            Act<DT>::store(const_cast<uint8_t*>(p.ring_k), slot_off + d, x[i]);
            reinterpret_cast<uint16_t*>(const_cast<uint8_t*>(p.ring_v))[slot_off + d] = vbits;
        }
    }
    __syncthreads();

    const int g = lane >> 2, c = lane & 3;
    const int rg = rho16(g), kA = rho16(2 * c), kB = kA ^ 4;
    uint32_t qb0[8], qb1[8];
#pragma unroll
    for (int t = 0; t < 8; t++) {
        const int m = t >> 1, e = t & 1;
        const int d0 = 64 * (m >> 1) + 8 * (c + 4 * (m & 1)) + 4 * e;
        qb0[t] = *reinterpret_cast<const uint32_t*>(&qs[g][d0]);
        qb1[t] = *reinterpret_cast<const uint32_t*>(&qs[g][d0 + 2]);
    }

    // ---- S^T = K Q^T for the warp's 32 rows
    float s[2][4];
#pragma unroll
    for (int step = 0; step < 2; step++) {
        s[step][0] = s[step][1] = s[step][2] = s[step][3] = 0.0f;
        const int r0 = warp * 32 + step * 16 + rg;
#pragma unroll
        for (int m = 0; m < 4; m++) {
            const uint8_t* base = Kt + (m >> 1) * (BLK * 128) + r0 * 128 + (((c + 4 * (m & 1)) ^ rg) << 4);
            const uint4 x0 = *reinterpret_cast<const uint4*>(base);
            const uint4 x1 = *reinterpret_cast<const uint4*>(base + 8 * 128);
            mma16<DT>(s[step], x0.x, x1.x, x0.y, x1.y, qb0[2 * m], qb1[2 * m]);
            mma16<DT>(s[step], x0.z, x1.z, x0.w, x1.w, qb0[2 * m + 1], qb1[2 * m + 1]);
        }
    }
    // softmax over the warp's rows: lane holds rows r0, r0 + 8 of each step, heads 2c and 2c + 1
    const float scale = rsqrtf(float(HD));
    bool valid[2][2];
    float m0 = NEG_BIG, m1 = NEG_BIG;
#pragma unroll
    for (int step = 0; step < 2; step++) {
        const int r0 = warp * 32 + step * 16 + rg;
        valid[step][0] = j0 + r0 < count;
        valid[step][1] = j0 + r0 + 8 < count;
#pragma unroll
        for (int e = 0; e < 4; e++) {
            s[step][e] = valid[step][e >> 1] ? s[step][e] * scale : NEG_BIG;
        }
        m0 = fmaxf(m0, fmaxf(s[step][0], s[step][2]));
        m1 = fmaxf(m1, fmaxf(s[step][1], s[step][3]));
    }
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
        m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, o));
        m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, o));
    }
    float l0 = 0.0f, l1 = 0.0f;
    float OT[8][4];
#pragma unroll
    for (int i = 0; i < 8; i++) OT[i][0] = OT[i][1] = OT[i][2] = OT[i][3] = 0.0f;
#pragma unroll
    for (int step = 0; step < 2; step++) {
        float pw[4];
#pragma unroll
        for (int e = 0; e < 4; e++) pw[e] = valid[step][e >> 1] ? __expf(s[step][e] - ((e & 1) ? m1 : m0)) : 0.0f;
        l0 += pw[0] + pw[2];
        l1 += pw[1] + pw[3];
        const int R0 = warp * 32 + step * 16;
        const uint8_t* vA = Vt + (R0 + kA) * 128 + ((g ^ kA) << 4);
        const uint8_t* vB = Vt + (R0 + kB) * 128 + ((g ^ kB) << 4);
        uint4 A[2], B[2], C[2], D[2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            A[h] = *reinterpret_cast<const uint4*>(vA + h * (BLK * 128));
            B[h] = *reinterpret_cast<const uint4*>(vB + h * (BLK * 128));
            C[h] = *reinterpret_cast<const uint4*>(vA + h * (BLK * 128) + 8 * 128);
            D[h] = *reinterpret_cast<const uint4*>(vB + h * (BLK * 128) + 8 * 128);
        }
        // P^T as B fragments; for bf16 P is split hi + lo so that its rounding stays below 2^-16
        const uint32_t pb0 = movmatrix_trans16(pack_act2<DT>(pw[0], pw[1]));
        const uint32_t pb1 = movmatrix_trans16(pack_act2<DT>(pw[2], pw[3]));
        uint32_t pl0 = 0, pl1 = 0;
        if (DT == EMBLA_BF16) {
            float lo[4];
#pragma unroll
            for (int e = 0; e < 4; e++) lo[e] = pw[e] - Act<EMBLA_BF16>::round(pw[e]);
            pl0 = movmatrix_trans16(pack_act2<DT>(lo[0], lo[1]));
            pl1 = movmatrix_trans16(pack_act2<DT>(lo[2], lo[3]));
        }
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int wi = i >> 1;
            const uint32_t sel = (i & 1) ? 0x7632 : 0x5410;
            const uint32_t a0 = __byte_perm(word4(A[0], wi), word4(B[0], wi), sel);
            const uint32_t a1 = __byte_perm(word4(A[1], wi), word4(B[1], wi), sel);
            const uint32_t a2 = __byte_perm(word4(C[0], wi), word4(D[0], wi), sel);
            const uint32_t a3 = __byte_perm(word4(C[1], wi), word4(D[1], wi), sel);
            mma16<DT>(OT[i], a0, a1, a2, a3, pb0, pb1);
            if (DT == EMBLA_BF16) mma16<DT>(OT[i], a0, a1, a2, a3, pl0, pl1);
        }
    }
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
        l0 += __shfl_xor_sync(0xffffffffu, l0, o);
        l1 += __shfl_xor_sync(0xffffffffu, l1, o);
    }

    // ---- merge the 4 warps (the K tile is free now)
    __syncthreads();
    float(*red)[8][HD] = reinterpret_cast<float(*)[8][HD]>(Kt);
    float(*redm)[8] = reinterpret_cast<float(*)[8]>(Kt + 4 * 8 * HD * 4);
    float(*redl)[8] = redm + 4;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        red[warp][2 * c][8 * g + i] = OT[i][0];
        red[warp][2 * c + 1][8 * g + i] = OT[i][1];
        red[warp][2 * c][64 + 8 * g + i] = OT[i][2];
        red[warp][2 * c + 1][64 + 8 * g + i] = OT[i][3];
    }
    if (g == 0) {
        redm[warp][2 * c] = m0;
        redm[warp][2 * c + 1] = m1;
        redl[warp][2 * c] = l0;
        redl[warp][2 * c + 1] = l1;
    }
    __syncthreads();
    const int pair = b * p.n_kv_heads + kvh;
    float* part = p.partials + (size_t(pair) * p.max_chunks + chunk) * p.G * A16_PART;
    for (int idx = tid; idx < p.G * HD; idx += A16_THREADS) {
        const int hh = idx >> 7, d = idx & 127;
        float M = NEG_BIG;
#pragma unroll
        for (int w = 0; w < 4; w++) M = fmaxf(M, redm[w][hh]);
        float L = 0.0f, num = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; w++) {
            const float f = __expf(redm[w][hh] - M);
            L += redl[w][hh] * f;
            num += red[w][hh][d] * f;
        }
        if (nch == 1) {
            Act<DT>::store(p.o, size_t(b) * p.o_stride + size_t(kvh * p.G + hh) * HD + d, num / L);
        } else {
            part[hh * A16_PART + d] = num;
            if (d == 0) {
                part[hh * A16_PART + HD] = M;
                part[hh * A16_PART + HD + 1] = L;
            }
        }
    }
    if (nch == 1) return;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const int prev = atomicAdd(&p.counters[pair], 1);
        s_last = prev == nch - 1;
        if (s_last) p.counters[pair] = 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const float* base = p.partials + size_t(pair) * p.max_chunks * p.G * A16_PART;
    for (int idx = tid; idx < p.G * HD; idx += A16_THREADS) {
        const int hh = idx >> 7, d = idx & 127;
        float M = NEG_BIG;
        for (int cc = 0; cc < nch; cc++) M = fmaxf(M, __ldcg(base + (size_t(cc) * p.G + hh) * A16_PART + HD));
        float L = 0.0f, num = 0.0f;
        for (int cc = 0; cc < nch; cc++) {
            const float* q2 = base + (size_t(cc) * p.G + hh) * A16_PART;
            const float f = __expf(__ldcg(q2 + HD) - M);
            L += __ldcg(q2 + HD + 1) * f;
            num += __ldcg(q2 + d) * f;
        }
        Act<DT>::store(p.o, size_t(b) * p.o_stride + size_t(kvh * p.G + hh) * HD + d, num / L);
    }
}

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

template <int MODE>
static EmblaStatus launch_attn16(EmblaAttn* ctx, Attn16Params& p, int batch, int max_rows, cudaStream_t s) {
    constexpr size_t smem = 1024 + 2 * A16_TILE + 8 * HD * 2;
    p.partials = ctx->partials;
    p.counters = ctx->counters;
    p.G = ctx->cfg.n_q_heads / ctx->cfg.n_kv_heads;
    p.n_kv_heads = ctx->cfg.n_kv_heads;
    p.max_chunks = (max_rows + BLK - 1) / BLK;
    if (long(batch) * p.n_kv_heads * p.max_chunks > ctx->partial_slots)
        EMBLA_FAIL(EMBLA_BAD_ARG, "attention scratch too small: %d sequences x %d chunks", batch, p.max_chunks);
    fill_rope_freq(p.rope_freq);
    dim3 grid(p.max_chunks, p.n_kv_heads, batch);
    static bool configured[2][64] = {};
    const bool bf = ctx->cfg.act_dtype == EMBLA_BF16;
    auto kern = bf ? attn16_decode_kernel<EMBLA_BF16, MODE> : attn16_decode_kernel<EMBLA_F16, MODE>;
    if (!configured[bf][ctx->device & 63]) {
        EMBLA_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        configured[bf][ctx->device & 63] = true;
    }
    kern<<<grid, A16_THREADS, smem, s>>>(p);
    EMBLA_CUDA_TRY(cudaGetLastError());
    return EMBLA_OK;
}

extern "C" EmblaStatus embla_attn_sparse_decode(EmblaAttn* ctx, const EmblaKVPool* pool, const EmblaKVView* view,
                                                const EmblaQuery* q, const uint32_t* idx_dev, void* o_dev,
                                                int64_t o_stride, void* stream) {
    if (!ctx || !pool || !view || !o_dev) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_sparse_decode: null argument");
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

extern "C" EmblaStatus embla_sliding_write(EmblaAttn* ctx, const EmblaRing* ring, const int32_t* pos0_dev, int32_t batch,
                                           int32_t n_tokens, const void* k_dev, const void* v_dev, int64_t token_stride,
                                           int64_t seq_stride, int32_t prenormed, const void* kgain_dev, void* stream) {
    if (!ctx || !ring || !ring->k_dev || !ring->v_dev || !pos0_dev || !k_dev || !v_dev)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_sliding_write: null argument");
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
    if (EmblaStatus st = check_query("embla_attn_sliding_decode", q)) return st;
    if (batch <= 0 || batch > ctx->cfg.max_batch || ring->window <= 0 || ring->window > ring->ring)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_sliding_decode: batch %d, window %d, ring %d", batch, ring->window, ring->ring);
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
