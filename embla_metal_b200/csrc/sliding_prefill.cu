// Prefill-chunk attention of the sliding layers: every new token attends its last `window` positions,
// all already in the ring (embla_sliding_write for the whole chunk first, as the reference runs
// kv_sliding_b before the attention, Sources/EmblaMetal/Prefill.swift:291-313). Replaces attn_sliding_b /
// attn_sliding8_b (Sources/EmblaMetal/Kernels/prefill.metal:129-180, 439-548).
//
// Like attn_sliding8_b, one CTA takes the 8 query rows that share a window — 8 / G consecutive tokens of
// one kv head's G query heads — and walks the union of their windows in tiles of 128 ring rows
// (16-byte cp.async, swizzled tiles). S^T = K Q^T and O^T = V^T P^T are m16n8k16 tensor tiles with the
// 8 query rows as the N columns; each row is masked to its own window, the softmax is online per warp
// (running max and sum per column, O rescaled when the max grows) and the 4 warps merge at the end.
// This version re-reads the window for every 8 rows (it lives in L2); a tcgen05 variant with 128-token
// tiles is the follow-up.
#include "attn16_common.cuh"
#include "sliding_prefill_tc.cuh"

namespace embla {

constexpr int SP_THREADS = 128;
constexpr int SP_TILE = BLK * HD * 2;

struct SlidingPrefillParams {
    const uint8_t* ring_k;
    const uint8_t* ring_v;
    const int32_t* pos0;
    const void* q;
    const void* g1;
    void* o;
    int64_t q_token_stride, q_seq_stride, o_token_stride, o_seq_stride, ring_stride;
    int n_tokens, n_kv_heads, G, prenormed, ring, window;
    float rope_freq[32];
};

template <int DT>
__global__ void __launch_bounds__(SP_THREADS) sliding_prefill_kernel(const SlidingPrefillParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* Kt = smem;
    uint8_t* Vt = smem + SP_TILE;
    uint16_t(*qs)[HD] = reinterpret_cast<uint16_t(*)[HD]>(smem + 2 * SP_TILE);   // [8 columns][128]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kvh = blockIdx.y, b = blockIdx.z;
    const int tpc = 8 / p.G;                          // tokens per CTA
    const int t0 = blockIdx.x * tpc;
    const int p0 = p.pos0[b];
    const int ntok = min(tpc, p.n_tokens - t0);       // valid tokens of this CTA
    const int pos_a = p0 + t0, pos_z = pos_a + ntok - 1;
    const int lo = max(0, pos_a - p.window + 1);
    const int ntiles = (pos_z - lo) / BLK + 1;

    // ---- the 8 query rows: column n = token n / G, head n % G (norm + RoPE at the token's position)
    for (int n = warp; n < 8; n += SP_THREADS / 32) {
        const int t = n / p.G, hh = n % p.G;
        float x[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (t < ntok) {
            const size_t off = size_t(b) * p.q_seq_stride + size_t(t0 + t) * p.q_token_stride + size_t(kvh * p.G + hh) * HD;
#pragma unroll
            for (int i = 0; i < 4; i++) x[i] = Act<DT>::load(p.q, off + lane + 32 * i);
            if (!p.prenormed) norm_rope_round<DT>(x, p.g1, p.g1, 1, pos_a + t, p.rope_freq, lane);
        }
#pragma unroll
        for (int i = 0; i < 4; i++) Act<DT>::store(&qs[n][0], lane + 32 * i, x[i]);
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
    // this lane's two columns (2c, 2c + 1): their positions; a missing token gets position -1 (sees nothing)
    const int tok0 = (2 * c) / p.G, tok1 = (2 * c + 1) / p.G;
    const int pc0 = tok0 < ntok ? pos_a + tok0 : -1, pc1 = tok1 < ntok ? pos_a + tok1 : -1;
    const float scale = rsqrtf(float(HD));
    float m0 = NEG_BIG, m1 = NEG_BIG, l0 = 0.0f, l1 = 0.0f;
    float OT[8][4];
#pragma unroll
    for (int i = 0; i < 8; i++) OT[i][0] = OT[i][1] = OT[i][2] = OT[i][3] = 0.0f;

    for (int tile = 0; tile < ntiles; tile++) {
        const int kbase = lo + tile * BLK;            // position of the tile's row 0
        {
            const int ch = tid & 15, half = ch >> 3, cc = ch & 7;
#pragma unroll 4
            for (int it = 0; it < 16; it++) {
                const int key = it * 8 + (tid >> 4), kp = kbase + key;
                const bool valid = kp <= pos_z;
                const int slot = valid ? kp % p.ring : 0;
                const size_t off = (size_t(b) * p.ring_stride + (size_t(kvh) * p.ring + slot) * HD) * 2 + ch * 16;
                const int dst = half * (BLK * 128) + key * 128 + ((cc ^ (key & 7)) << 4);
                cp_async16(Kt + dst, p.ring_k + off, valid);
                cp_async16(Vt + dst, p.ring_v + off, valid);
            }
        }
        cp_async_wait_all();
        __syncthreads();

        float s[2][4];
        bool ok[2][4];
        float tm0 = NEG_BIG, tm1 = NEG_BIG;
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
            // rows r0 (elements 0, 1) and r0 + 8 (elements 2, 3); columns 2c (even elements) and 2c + 1
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int kp = kbase + r0 + 8 * (e >> 1), pc = (e & 1) ? pc1 : pc0;
                ok[step][e] = kp <= pc && kp > pc - p.window;
                s[step][e] = ok[step][e] ? s[step][e] * scale : NEG_BIG;
            }
            tm0 = fmaxf(tm0, fmaxf(s[step][0], s[step][2]));
            tm1 = fmaxf(tm1, fmaxf(s[step][1], s[step][3]));
        }
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
            tm0 = fmaxf(tm0, __shfl_xor_sync(0xffffffffu, tm0, o));
            tm1 = fmaxf(tm1, __shfl_xor_sync(0xffffffffu, tm1, o));
        }
        const float n0 = fmaxf(m0, tm0), n1 = fmaxf(m1, tm1);
        const float f0 = __expf(m0 - n0), f1 = __expf(m1 - n1);
        m0 = n0;
        m1 = n1;
        l0 *= f0;
        l1 *= f1;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            OT[i][0] *= f0;
            OT[i][1] *= f1;
            OT[i][2] *= f0;
            OT[i][3] *= f1;
        }
#pragma unroll
        for (int step = 0; step < 2; step++) {
            float pw[4];
#pragma unroll
            for (int e = 0; e < 4; e++) pw[e] = ok[step][e] ? __expf(s[step][e] - ((e & 1) ? m1 : m0)) : 0.0f;
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
            const uint32_t pb0 = movmatrix_trans16(pack_act2<DT>(pw[0], pw[1]));
            const uint32_t pb1 = movmatrix_trans16(pack_act2<DT>(pw[2], pw[3]));
            uint32_t pl0 = 0, pl1 = 0;
            if (DT == EMBLA_BF16) {   // P split hi + lo so that its rounding stays below 2^-16
                float lo4[4];
#pragma unroll
                for (int e = 0; e < 4; e++) lo4[e] = pw[e] - Act<EMBLA_BF16>::round(pw[e]);
                pl0 = movmatrix_trans16(pack_act2<DT>(lo4[0], lo4[1]));
                pl1 = movmatrix_trans16(pack_act2<DT>(lo4[2], lo4[3]));
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
        __syncthreads();   // the tiles are overwritten by the next round of copies
    }
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
        l0 += __shfl_xor_sync(0xffffffffu, l0, o);
        l1 += __shfl_xor_sync(0xffffffffu, l1, o);
    }

    // ---- merge the 4 warps and write the 8 rows
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
    for (int idx = tid; idx < 8 * HD; idx += SP_THREADS) {
        const int n = idx >> 7, d = idx & 127;
        const int t = n / p.G, hh = n % p.G;
        if (t >= ntok) continue;
        float M = NEG_BIG;
#pragma unroll
        for (int w = 0; w < 4; w++) M = fmaxf(M, redm[w][n]);
        float L = 0.0f, num = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; w++) {
            const float f = __expf(redm[w][n] - M);
            L += redl[w][n] * f;
            num += red[w][n][d] * f;
        }
        Act<DT>::store(p.o, size_t(b) * p.o_seq_stride + size_t(t0 + t) * p.o_token_stride + size_t(kvh * p.G + hh) * HD + d, num / L);
    }
}

}  // namespace embla

using namespace embla;

extern "C" EmblaStatus embla_attn_sliding_prefill(EmblaAttn* ctx, const EmblaRing* ring, const int32_t* pos0_dev, int32_t batch,
                                                  int32_t n_tokens, const EmblaQuery* q, int64_t q_token_stride, void* o_dev,
                                                  int64_t o_token_stride, int64_t o_seq_stride, void* stream) {
    if (!ctx || !ring || !ring->k_dev || !ring->v_dev || !pos0_dev || !q || !q->q_dev || !o_dev)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_sliding_prefill: null argument");
    EMBLA_CHECK_DEVICE("embla_attn_sliding_prefill", ctx, static_cast<const EmblaKVPool*>(nullptr));
    if (batch <= 0 || n_tokens <= 0 || ring->window <= 0 || ring->window + n_tokens > ring->ring)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_sliding_prefill: the ring (%d slots) must hold the window (%d) and the chunk (%d tokens)",
                   ring->ring, ring->window, n_tokens);
    if (!q->prenormed && (q->ng != 1 || !q->g1_dev))
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_sliding_prefill: the fused head norm takes the query gain (ng = 1)");
    const int G = ctx->cfg.n_q_heads / ctx->cfg.n_kv_heads;
    if (G != 1 && G != 2 && G != 4 && G != 8)
        EMBLA_FAIL(EMBLA_UNSUPPORTED, "embla_attn_sliding_prefill: %d query heads per kv head (1, 2, 4 or 8)", G);
    SlidingPrefillParams p;
    p.ring_k = static_cast<const uint8_t*>(ring->k_dev);
    p.ring_v = static_cast<const uint8_t*>(ring->v_dev);
    p.pos0 = pos0_dev;
    p.q = q->q_dev;
    p.g1 = q->g1_dev;
    p.o = o_dev;
    p.q_token_stride = q_token_stride;
    p.q_seq_stride = q->q_stride;
    p.o_token_stride = o_token_stride;
    p.o_seq_stride = o_seq_stride;
    p.ring_stride = ring->seq_stride;
    p.n_tokens = n_tokens;
    p.n_kv_heads = ctx->cfg.n_kv_heads;
    p.G = G;
    p.prenormed = q->prenormed;
    p.ring = ring->ring;
    p.window = ring->window;
    fill_rope_freq(p.rope_freq);
    // Whole chunks over rings of a multiple of 128 slots run on the tcgen05 kernel (sliding_prefill_tc.cu); short chunks
    // and other rings take the kernel below.
    if (n_tokens >= 64 && ring->ring % BLK == 0 && ring->seq_stride % 8 == 0 &&
        reinterpret_cast<uintptr_t>(ring->k_dev) % 16 == 0 && reinterpret_cast<uintptr_t>(ring->v_dev) % 16 == 0 &&
        q_token_stride % 8 == 0 && q->q_stride % 8 == 0 && reinterpret_cast<uintptr_t>(q->q_dev) % 16 == 0 && o_token_stride % 8 == 0 && o_seq_stride % 8 == 0 &&
        reinterpret_cast<uintptr_t>(o_dev) % 16 == 0) {
        SlidingTcParams t = {};
        t.pos0 = pos0_dev;
        t.q = q->q_dev;
        t.g1 = q->g1_dev;
        t.o = o_dev;
        t.ctl = kernel_ctl(ctx);
        t.q_token_stride = q_token_stride;
        t.q_seq_stride = q->q_stride;
        t.o_token_stride = o_token_stride;
        t.o_seq_stride = o_seq_stride;
        t.n_tokens = n_tokens;
        t.n_kv_heads = ctx->cfg.n_kv_heads;
        t.G = G;
        t.prenormed = q->prenormed;
        t.ring = ring->ring;
        t.window = ring->window;
        fill_rope_freq(t.rope_freq);
        return launch_sliding_prefill_tc(ctx, ring, t, batch, static_cast<cudaStream_t>(stream));
    }
    constexpr size_t smem = 1024 + 2 * SP_TILE + 8 * HD * 2;
    const int tpc = 8 / G;
    dim3 grid((n_tokens + tpc - 1) / tpc, p.n_kv_heads, batch);
    const bool bf = ctx->cfg.act_dtype == EMBLA_BF16;
    auto kern = bf ? sliding_prefill_kernel<EMBLA_BF16> : sliding_prefill_kernel<EMBLA_F16>;
    static bool configured[2][64] = {};
    if (!configured[bf][ctx->device & 63]) {
        EMBLA_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        configured[bf][ctx->device & 63] = true;
    }
    kern<<<grid, SP_THREADS, smem, static_cast<cudaStream_t>(stream)>>>(p);
    EMBLA_CUDA_TRY(cudaGetLastError());
    return EMBLA_OK;
}
