// Decode attention of sparse layers that read the preceding full layer's int8 cache, as the reference's own
// model does (Sources/EmblaMetal/Engine.swift:461-462): softmax over every key of a sequence with at most 1152
// keys, else over the rows idx[kv head][0..1151] that embla_select_keys wrote from the full layer's scores.
// Replaces attn_sparse8 / attn_sparse_short (Sources/EmblaMetal/Kernels/attention.metal:448-584, 593-645).
//
// Same shape as the 16-bit gather kernel (one CTA = 128 rows of one (sequence, kv head), 16-byte cp.async
// gathers into swizzled tiles, exact softmax inside the CTA, (max, sum, acc) partials merged by the last CTA),
// with the int8 arithmetic of the full-layer decode kernel: codes widened exactly to fp16 in registers,
// S^T = K Q^T and O^T = V^T P^T as m16n8k16 tiles, key scale on S, value scale folded into P.
#include "attn16_common.cuh"

namespace embla {

constexpr int S8_THREADS = 128;
constexpr int S8_PART = HD + 4;

struct Sparse8Params {
    const uint8_t* pool;
    const int32_t* block_table;
    const uint32_t* idx;
    const int32_t* seq_lens;
    const void* q;
    const void* g1;
    const void* g2;
    void* o;
    float* partials;
    int* counters;
    KernelCtl ctl;
    int64_t q_stride, o_stride;
    size_t page_bytes;
    int table_stride, layer, n_layers, n_kv_heads, G, prenormed, ng, max_chunks;
};

template <int DT, int SB>
__global__ void __launch_bounds__(S8_THREADS) sparse8_decode_kernel(const Sparse8Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* Kt = smem;                                   // [128 rows][128 B] int8, chunk ^ (row % 8)
    uint8_t* Vt = smem + CODE_BYTES;
    float* ksc = reinterpret_cast<float*>(smem + 2 * CODE_BYTES);   // [128] key scales / sqrt(D)
    float* vsc = ksc + BLK;                                          // [128] value scales
    __half(*qh)[HD] = reinterpret_cast<__half(*)[HD]>(vsc + BLK);    // [8][128]
    __shared__ int s_last;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int chunk = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    trace_first(p.ctl.trace, 0);
    const int S = p.seq_lens[b];   // (read ahead of the wait: nothing on the GPU writes the sequence lengths)
    pdl_wait();
    pdl_launch_dependents();
    trace_first(p.ctl.trace, 1);
    const bool selecting = S > EMBLA_TOPK + EMBLA_RECENT;
    const int count = selecting ? EMBLA_TOPK + EMBLA_RECENT : S;
    const int nch = (count + BLK - 1) / BLK;
    if (chunk >= nch) return;
    const int j0 = chunk * BLK;

    // ---- gather this chunk's code rows (8 chunks of 16 bytes a row and side) and their scales
    {
        const int ch = tid & 7;
#pragma unroll
        for (int it = 0; it < 8; it++) {
            const int key = it * 16 + (tid >> 3), j = j0 + key;
            const bool valid = j < count;
            int row = valid ? j : 0;
            if (selecting && valid) row = int(p.idx[(size_t(b) * p.n_kv_heads + kvh) * (EMBLA_TOPK + EMBLA_RECENT) + j]);
            const int block = p.block_table[size_t(b) * p.table_stride + (row >> 7)];
            const uint8_t* page = p.pool + ((size_t(block) * p.n_layers + p.layer) * p.n_kv_heads + kvh) * p.page_bytes;
            const uint8_t* ksrc = page + (row & 127) * HD + ch * 16;
            const int dst = key * 128 + ((ch ^ (key & 7)) << 4);
            cp_async16(Kt + dst, ksrc, valid);
            cp_async16(Vt + dst, ksrc + CODE_BYTES, valid);
            if (ch == 0) {
                const uint8_t* sc = page + 2 * CODE_BYTES;
                float ks = 0.0f, vs = 0.0f;
                if (valid) {
                    ks = SB == 4 ? reinterpret_cast<const float*>(sc)[row & 127] : __half2float(reinterpret_cast<const __half*>(sc)[row & 127]);
                    vs = SB == 4 ? reinterpret_cast<const float*>(sc + BLK * SB)[row & 127]
                                 : __half2float(reinterpret_cast<const __half*>(sc + BLK * SB)[row & 127]);
                }
                ksc[key] = ks * rsqrtf(float(HD));
                vsc[key] = vs;
            }
        }
    }
    // ---- the kv head's queries (head norm with both gains) as fp16 while the rows arrive
    for (int hh = warp; hh < 8; hh += S8_THREADS / 32) {
        float x[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (hh < p.G) {
            const size_t off = size_t(b) * p.q_stride + size_t(kvh * p.G + hh) * HD;
#pragma unroll
            for (int i = 0; i < 4; i++) x[i] = Act<DT>::load(p.q, off + lane + 32 * i);
            if (!p.prenormed) norm_rope_round<DT>(x, p.g1, p.g2, p.ng, -1, nullptr, lane);
        }
#pragma unroll
        for (int i = 0; i < 4; i++) qh[hh][lane + 32 * i] = __float2half_rn(x[i]);
    }
    cp_async_wait_all();
    __syncthreads();

    const int g = lane >> 2, c = lane & 3;
    const int rg = rho16(g), kA = rho16(2 * c), kB = kA ^ 4;
    uint32_t qb0[8], qb1[8];
#pragma unroll
    for (int t = 0; t < 8; t++) {
        const int d0 = (t < 4) ? 16 * c + 4 * t : 64 + 16 * c + 4 * (t - 4);
        qb0[t] = *reinterpret_cast<const uint32_t*>(&qh[g][d0]);
        qb1[t] = *reinterpret_cast<const uint32_t*>(&qh[g][d0 + 2]);
    }
    // ---- S^T = K Q^T for the warp's 32 rows; lane holds rows r0, r0 + 8 of each step, heads 2c and 2c + 1
    float s[2][4];
    bool valid[2][2];
    float m0 = NEG_BIG, m1 = NEG_BIG;
#pragma unroll
    for (int step = 0; step < 2; step++) {
        s[step][0] = s[step][1] = s[step][2] = s[step][3] = 0.0f;
        const int r0 = warp * 32 + step * 16 + rg;
        const uint8_t* k0 = Kt + r0 * 128;
        const uint4 lo0 = *reinterpret_cast<const uint4*>(k0 + ((c ^ rg) << 4));
        const uint4 hi0 = *reinterpret_cast<const uint4*>(k0 + (((c + 4) ^ rg) << 4));
        const uint4 lo1 = *reinterpret_cast<const uint4*>(k0 + 8 * 128 + ((c ^ rg) << 4));
        const uint4 hi1 = *reinterpret_cast<const uint4*>(k0 + 8 * 128 + (((c + 4) ^ rg) << 4));
        const uint32_t w0[8] = {lo0.x, lo0.y, lo0.z, lo0.w, hi0.x, hi0.y, hi0.z, hi0.w};
        const uint32_t w1[8] = {lo1.x, lo1.y, lo1.z, lo1.w, hi1.x, hi1.y, hi1.z, hi1.w};
#pragma unroll
        for (int t = 0; t < 8; t++) {
            const uint32_t x0 = w0[t] ^ 0x80808080u, x1 = w1[t] ^ 0x80808080u;
            mma_16816(s[step], h2_from_biased_bytes(x0, 0x4140), h2_from_biased_bytes(x1, 0x4140),
                      h2_from_biased_bytes(x0, 0x4342), h2_from_biased_bytes(x1, 0x4342), qb0[t], qb1[t]);
        }
        valid[step][0] = j0 + r0 < count;
        valid[step][1] = j0 + r0 + 8 < count;
        const float f0 = ksc[r0], f1 = ksc[r0 + 8];
        s[step][0] = valid[step][0] ? s[step][0] * f0 : NEG_BIG;
        s[step][1] = valid[step][0] ? s[step][1] * f0 : NEG_BIG;
        s[step][2] = valid[step][1] ? s[step][2] * f1 : NEG_BIG;
        s[step][3] = valid[step][1] ? s[step][3] * f1 : NEG_BIG;
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
        const int R0 = warp * 32 + step * 16, r0 = R0 + rg;
        float pw[4];
#pragma unroll
        for (int e = 0; e < 4; e++) pw[e] = valid[step][e >> 1] ? __expf(s[step][e] - ((e & 1) ? m1 : m0)) : 0.0f;
        l0 += pw[0] + pw[2];
        l1 += pw[1] + pw[3];
        const float v0 = vsc[r0], v1 = vsc[r0 + 8];
        const uint32_t pb0 = movmatrix_trans16(pack_h2(pw[0] * v0, pw[1] * v0));
        const uint32_t pb1 = movmatrix_trans16(pack_h2(pw[2] * v1, pw[3] * v1));
        const uint8_t* vA = Vt + (R0 + kA) * 128 + ((g ^ kA) << 4);
        const uint8_t* vB = Vt + (R0 + kB) * 128 + ((g ^ kB) << 4);
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
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
        l0 += __shfl_xor_sync(0xffffffffu, l0, o);
        l1 += __shfl_xor_sync(0xffffffffu, l1, o);
    }

    // ---- merge the 4 warps (the K tile is free now); O^T tile i: dims 16g + i (rows g) and 16g + 8 + i (rows g + 8)
    __syncthreads();
    float(*red)[8][HD] = reinterpret_cast<float(*)[8][HD]>(Kt);
    float(*redm)[8] = reinterpret_cast<float(*)[8]>(Vt);
    float(*redl)[8] = redm + 4;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        red[warp][2 * c][16 * g + i] = OT[i][0];
        red[warp][2 * c + 1][16 * g + i] = OT[i][1];
        red[warp][2 * c][16 * g + 8 + i] = OT[i][2];
        red[warp][2 * c + 1][16 * g + 8 + i] = OT[i][3];
    }
    if (g == 0) {
        redm[warp][2 * c] = m0;
        redm[warp][2 * c + 1] = m1;
        redl[warp][2 * c] = l0;
        redl[warp][2 * c + 1] = l1;
    }
    __syncthreads();
    const int pair = b * p.n_kv_heads + kvh;
    float* part = p.partials + (size_t(pair) * p.max_chunks + chunk) * p.G * S8_PART;
    for (int idx = tid; idx < p.G * HD; idx += S8_THREADS) {
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
            part[hh * S8_PART + d] = num;
            if (d == 0) {
                part[hh * S8_PART + HD] = M;
                part[hh * S8_PART + HD + 1] = L;
            }
        }
    }
    trace_last(p.ctl.trace, 2);
    if (nch == 1) {
        trace_last(p.ctl.trace, 3);
        return;
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const int prev = atomicAdd(&p.counters[pair], 1);
        s_last = prev == nch - 1;
        if (s_last) p.counters[pair] = 0;
    }
    __syncthreads();
    if (!s_last) {
        trace_last(p.ctl.trace, 3);
        return;
    }
    __threadfence();
    // the pair's partials (contiguous: [chunk][head][128 sums, max, sum]; at most 9 chunks x 8 heads: 38 KB) into the
    // tile area in one batch of loads, then the merge in chunk order from shared memory
    const float* gbase = p.partials + size_t(pair) * p.max_chunks * p.G * S8_PART;
    float* sbase = reinterpret_cast<float*>(smem);
    stage_from_global<S8_THREADS>(reinterpret_cast<float4*>(sbase), reinterpret_cast<const float4*>(gbase), nch * p.G * (S8_PART / 4), tid);
    __syncthreads();
    for (int idx = tid; idx < p.G * HD; idx += S8_THREADS) {
        const int hh = idx >> 7, d = idx & 127;
        float M = NEG_BIG;
        for (int cc = 0; cc < nch; cc++) M = fmaxf(M, sbase[(cc * p.G + hh) * S8_PART + HD]);
        float L = 0.0f, num = 0.0f;
        for (int cc = 0; cc < nch; cc++) {
            const float* q2 = sbase + (cc * p.G + hh) * S8_PART;
            const float f = __expf(q2[HD] - M);
            L += q2[HD + 1] * f;
            num += q2[d] * f;
        }
        Act<DT>::store(p.o, size_t(b) * p.o_stride + size_t(kvh * p.G + hh) * HD + d, num / L);
    }
    trace_last(p.ctl.trace, 3);
}

template <int DT, int SB>
static EmblaStatus launch_sparse8(EmblaAttn* ctx, const Sparse8Params& p, int batch, cudaStream_t s) {
    // tiles, scales and queries; the last CTA of a pair stages up to 9 chunks x 8 heads x 528 bytes of partials over them
    constexpr size_t smem = 1024 + 2 * CODE_BYTES + 2 * BLK * 4 + 8 * HD * 2 + 4096;
    static_assert(9 * 8 * S8_PART * 4 <= 2 * CODE_BYTES + 2 * BLK * 4 + 8 * HD * 2 + 4096, "partials do not fit the tile area");
    dim3 grid(p.max_chunks, p.n_kv_heads, batch);
    EMBLA_CUDA_TRY(launch_kernel(ctx->pdl, sparse8_decode_kernel<DT, SB>, grid, dim3(S8_THREADS), smem, s, p));
    EMBLA_CUDA_TRY(cudaGetLastError());
    (void)ctx;
    return EMBLA_OK;
}

}  // namespace embla

using namespace embla;

extern "C" EmblaStatus embla_attn_sparse_decode_int8(EmblaAttn* ctx, const EmblaKVPool* pool, const EmblaKVView* view,
                                                     const EmblaQuery* q, const uint32_t* idx_dev, void* o_dev,
                                                     int64_t o_stride, void* stream) {
    if (!ctx || !pool || !view || !q || !q->q_dev || !o_dev) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_sparse_decode_int8: null argument");
    EMBLA_CHECK_DEVICE("embla_attn_sparse_decode_int8", ctx, pool);
    if (pool->kv_dtype != EMBLA_KV_INT8) EMBLA_FAIL(EMBLA_UNSUPPORTED, "embla_attn_sparse_decode_int8: the pool is not int8");
    if (pool->n_kv_heads != ctx->cfg.n_kv_heads || view->layer < 0 || view->layer >= pool->n_layers)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_sparse_decode_int8: pool/layer mismatch");
    if (view->batch <= 0 || view->batch > ctx->cfg.max_batch || !view->block_table_dev || !view->seq_lens_dev)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_sparse_decode_int8: bad view (batch %d)", view->batch);
    if (!q->prenormed && (q->ng < 0 || q->ng > 2 || (q->ng >= 1 && !q->g1_dev) || (q->ng >= 2 && !q->g2_dev)))
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_sparse_decode_int8: ng %d without its gain vectors", q->ng);
    const int max_len = view->max_seq_len > 0 ? view->max_seq_len : ctx->cfg.max_context;
    if (max_len > EMBLA_TOPK + EMBLA_RECENT && !idx_dev)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_sparse_decode_int8: sequences past %d keys need the selected rows",
                   EMBLA_TOPK + EMBLA_RECENT);
    Sparse8Params p;
    p.pool = pool->base;
    p.block_table = view->block_table_dev;
    p.idx = idx_dev;
    p.seq_lens = view->seq_lens_dev;
    p.q = q->q_dev;
    p.g1 = q->g1_dev;
    p.g2 = q->g2_dev;
    p.o = o_dev;
    p.partials = ctx->partials;
    p.counters = ctx->counters;
    p.ctl = kernel_ctl(ctx);
    p.q_stride = q->q_stride;
    p.o_stride = o_stride;
    p.page_bytes = pool->page_bytes;
    p.table_stride = view->table_stride;
    p.layer = view->layer;
    p.n_layers = pool->n_layers;
    p.n_kv_heads = pool->n_kv_heads;
    p.G = ctx->cfg.n_q_heads / ctx->cfg.n_kv_heads;
    p.prenormed = q->prenormed;
    p.ng = q->ng;
    const int rows = max_len < EMBLA_TOPK + EMBLA_RECENT ? max_len : EMBLA_TOPK + EMBLA_RECENT;
    p.max_chunks = (rows + BLK - 1) / BLK;
    if (long(view->batch) * p.n_kv_heads * p.max_chunks > ctx->partial_slots)
        EMBLA_FAIL(EMBLA_BAD_ARG, "attention scratch too small: %d sequences x %d chunks", view->batch, p.max_chunks);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool bf = ctx->cfg.act_dtype == EMBLA_BF16, s4 = pool->scale_bytes == 4;
    if (bf) return s4 ? launch_sparse8<EMBLA_BF16, 4>(ctx, p, view->batch, s) : launch_sparse8<EMBLA_BF16, 2>(ctx, p, view->batch, s);
    return s4 ? launch_sparse8<EMBLA_F16, 4>(ctx, p, view->batch, s) : launch_sparse8<EMBLA_F16, 2>(ctx, p, view->batch, s);
}
