// The producer of a layer's q, k, v rows: the reference's 4-bit stacked GEMV (gemv / GemvRows,
// Sources/EmblaMetal/Kernels/gemv.metal:37-92, common.metal:105-152; dispatch Engine.swift:746-752) for a batch of tokens,
// with what the attention side otherwise does to the rows folded into its epilogue: for a full layer the head norm of q
// with its gains (head_norm, common.metal:30-41) and the quantised write of the current token's k and v into the paged
// int8 cache (kv_append + write_row8, attention.metal:113-140, common.metal:74-84). The attention launch that follows
// then takes prenormed queries and appends nothing.
//
// A weight row is 2048 four-bit values in 64 words of 16 bytes (word c, 32-bit part k, nibble n: column 32 c + 8 k + n)
// with one bfloat16 scale a and bias b per 64 columns: y = sum over words c of a(c / 2) * (sum nib * x) + b(c / 2) * (sum x).
// The products run on the tensor cores (mma.sync m16n8k16: a four-bit value is exact in fp16 and in bfloat16, so a weight
// word goes from its nibbles to an A fragment with a few integer operations, x is the B operand as it is stored): one
// accumulation per group of 64 columns in fp32, then a * (that) + b * (the group's sum of x) added to the output in fp32, as
// the reference adds them. A lane of the quad (g, c) takes byte c of each 32-bit part of the words of rows g and g + 8: two
// nibbles, the columns 2c, 2c + 1 (+ 8) of a k-step, which is the fragment layout with the columns in their natural
// order. Against the CPU restatement the outputs agree to the last place of the storage dtype or one step (the fp32 sums
// differ in order only); the fused and the plain epilogue share this arithmetic, so the cache bytes do not depend on
// which of them wrote them.
//   grid (head, token tile): a CTA computes the 128 rows of one head (of q, k or v) for up to 16 tokens, 16 rows a warp,
//   so the epilogue has whole heads in hand: norm, rounding, quantisation and the cache write are the device functions of
//   the append kernel. The weights (3.5 MB a layer at the benchmark's shape) are read once a token tile.
#include "attn16_common.cuh"
#include "kv_row.cuh"

namespace embla {

constexpr int QP_TOKENS = 16;     // tokens of a CTA
constexpr int QP_NT = QP_TOKENS / 8;   // n-tiles of 8 tokens
constexpr int QP_THREADS = 256;   // 8 warps x 16 rows = one head

struct QkvProjectParams {
    const uint4* w[3];            // q, k, v: words [rows][d_in / 32]
    const uint16_t* sc[3];        // bfloat16 scales [rows][d_in / 64]
    const uint16_t* bs[3];        // bfloat16 biases
    const void* x;                // [batch][x_stride] activation dtype
    void* qkv;                    // [batch][qkv_stride]: q heads, k heads, v heads
    const void* g1;
    const void* g2;
    uint8_t* pool;                // fused: the int8 pool of the layer's cache (else nullptr: k, v go to qkv as computed)
    const int32_t* block_table;
    const int32_t* seq_lens;      // fused: the token's position is seq_len - 1
    KernelCtl ctl;                // error word and wait limit
    float* resid;                 // o-projection: the fp32 residual rows [batch][qkv_stride] the outputs go (or are added) to
    int resid_add;
    uint8_t* ring_k;              // fused, sliding layer: the rings the token's k (normed with kgain, rotated) and v go to
    uint8_t* ring_v;
    const void* kgain;
    int64_t ring_stride;
    int ring;
    float rope_freq[32];
    int64_t x_stride, qkv_stride;
    size_t page_bytes;
    int d_in, batch, n_q_heads, n_kv_heads, ng, table_stride, layer, n_layers, scale_bytes, norm_k;
};

__device__ __forceinline__ float bf16_bits_to_float(uint16_t b) { return __uint_as_float(uint32_t(b) << 16); }

// The two nibbles of byte `c` of `part` as a pair of 16-bit floats (low nibble in the low half), exactly: their bits
// under the exponent of 1024 (fp16) or 128 (bfloat16), minus that.
template <int DT>
__device__ __forceinline__ uint32_t nibble_pair(uint32_t part, int c) {
    const uint32_t b = (part >> (8 * c)) & 0xFFu;
    const uint32_t bits = (b & 0x0Fu) | ((b & 0xF0u) << 12);
    if (DT == EMBLA_F16) {
        const uint32_t v = bits | 0x64006400u, m = 0x64006400u;
        const __half2 h = __hsub2(*reinterpret_cast<const __half2*>(&v), *reinterpret_cast<const __half2*>(&m));
        return *reinterpret_cast<const uint32_t*>(&h);
    }
    const uint32_t v = bits | 0x43004300u, m = 0x43004300u;
    const __nv_bfloat162 h = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&v), *reinterpret_cast<const __nv_bfloat162*>(&m));
    return *reinterpret_cast<const uint32_t*>(&h);
}

template <int DT>
__global__ void __launch_bounds__(QP_THREADS) qkv_project_kernel(const QkvProjectParams p) {
    extern __shared__ __align__(16) uint8_t qp_smem[];
    __shared__ uint64_t wbar;
    const int words = p.d_in / 32, groups = p.d_in / 64;
    const int xld = p.d_in + 8;                                  // 16-bit elements a token row of x (padded: no bank conflicts)
    const int wld = words * 16 + 16;                             // bytes a weight row in shared memory (padded likewise)
    uint16_t* xs16 = reinterpret_cast<uint16_t*>(qp_smem);       // [tokens][xld] as stored
    float* xsum = reinterpret_cast<float*>(qp_smem + size_t(QP_TOKENS) * xld * 2);   // [groups][tokens]: sum of x over the group
    uint16_t* wsc = reinterpret_cast<uint16_t*>(xsum + groups * QP_TOKENS);          // [128 rows][groups] bfloat16 scales, then the biases
    uint16_t* wbs = wsc + HD * groups;
    uint8_t* wsm = reinterpret_cast<uint8_t*>(wbs + HD * groups);                    // [128 rows][wld]: the head's weight words
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, c = lane & 3;
    const int head = blockIdx.x, tok0 = blockIdx.y * QP_TOKENS;
    const int ntok = min(QP_TOKENS, p.batch - tok0);
    const int seg = head < p.n_q_heads ? 0 : (head < p.n_q_heads + p.n_kv_heads ? 1 : 2);
    const int seg_head = seg == 0 ? head : (seg == 1 ? head - p.n_q_heads : head - p.n_q_heads - p.n_kv_heads);

    // ---- the head's 128 weight rows into shared memory, one bulk copy a row (a row is contiguous in global memory; read
    // straight from global by the lanes that use them, 16 bytes from 16 different rows an instruction, they kept the load
    // path busy for two thirds of the kernel)
    if (tid == 0) {
        mbar_init(&wbar, 1);
        fence_barrier_init();
        mbar_expect_tx(&wbar, uint32_t(HD) * words * 16);
    }
    __syncthreads();
    if (tid < HD) bulk_load_1d(wsm + tid * wld, p.w[seg] + (size_t(seg_head) * HD + tid) * words, uint32_t(words) * 16, &wbar);

    // ---- x of the tile's tokens as stored (16 bytes a thread and trip); rows past the batch are zeros
    {
        const int per_row = p.d_in / 8, total = QP_TOKENS * per_row;
        for (int i0 = tid; i0 < total; i0 += 8 * QP_THREADS) {      // eight loads of a thread in flight together
            uint4 v[8];
#pragma unroll
            for (int k = 0; k < 8; k++) {
                const int i = i0 + k * QP_THREADS, t = i / per_row, c8 = i % per_row;
                v[k] = make_uint4(0, 0, 0, 0);
                if (i < total && t < ntok)
                    v[k] = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.x) + size_t(tok0 + t) * p.x_stride + c8 * 8);
            }
#pragma unroll
            for (int k = 0; k < 8; k++) {
                const int i = i0 + k * QP_THREADS, t = i / per_row, c8 = i % per_row;
                if (i < total) *reinterpret_cast<uint4*>(xs16 + t * xld + c8 * 8) = v[k];
            }
        }
    }
    for (int i = tid; i < HD * groups; i += QP_THREADS) {      // (contiguous in global: the head's rows follow one another)
        wsc[i] = __ldg(p.sc[seg] + size_t(seg_head) * HD * groups + i);
        wbs[i] = __ldg(p.bs[seg] + size_t(seg_head) * HD * groups + i);
    }
    __syncthreads();
    for (int i = tid; i < groups * QP_TOKENS; i += QP_THREADS) {
        const int grp = i / QP_TOKENS, t = i % QP_TOKENS;
        uint4 v[8];                                      // the group's 64 values of the token: 128 bytes, loaded at once
#pragma unroll
        for (int k = 0; k < 8; k++) v[k] = *reinterpret_cast<const uint4*>(xs16 + t * xld + 64 * grp + 8 * k);
        float s = 0.0f;
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const uint32_t wv[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
#pragma unroll
            for (int e = 0; e < 4; e++) {
                if (DT == EMBLA_F16) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&wv[e]));
                    s += f.x;
                    s += f.y;
                } else {
                    s += __uint_as_float(wv[e] << 16);
                    s += __uint_as_float(wv[e] & 0xffff0000u);
                }
            }
        }
        xsum[grp * QP_TOKENS + t] = s;
    }
    __syncthreads();

    // ---- rows 16 warp + g and + 8 of the head; n-tiles of eight tokens
    const uint4* wr0 = reinterpret_cast<const uint4*>(wsm + (16 * warp + g) * wld);
    const uint4* wr1 = reinterpret_cast<const uint4*>(wsm + (16 * warp + g + 8) * wld);
    const uint16_t* sc0 = wsc + (16 * warp + g) * groups;
    const uint16_t* bs0 = wbs + (16 * warp + g) * groups;
    float acc[QP_NT][4];
#pragma unroll
    for (int j = 0; j < QP_NT; j++) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;
    const bool have_w = __all_sync(0xffffffffu, mbar_wait_bounded(p.ctl.wait_cycles, &wbar, 0));
    if (!have_w && lane == 0) atomicCAS(p.ctl.err, 0, ERR_WAIT_FULL);
    for (int grp = 0; grp < (have_w ? groups : 0); grp++) {
        float d[QP_NT][4];
#pragma unroll
        for (int j = 0; j < QP_NT; j++) d[j][0] = d[j][1] = d[j][2] = d[j][3] = 0.0f;
#pragma unroll
        for (int half = 0; half < 2; half++) {           // a word of 16 bytes: 32 columns, two k-steps
            const int w = 2 * grp + half;
            const uint4 u0 = wr0[w], u1 = wr1[w];
            const uint32_t pa[4] = {u0.x, u0.y, u0.z, u0.w}, pb[4] = {u1.x, u1.y, u1.z, u1.w};
#pragma unroll
            for (int s2 = 0; s2 < 2; s2++) {             // k-step: columns 32 w + 16 s2 .. + 15 (parts 2 s2 and 2 s2 + 1)
                const uint32_t a0 = nibble_pair<DT>(pa[2 * s2], c), a1 = nibble_pair<DT>(pb[2 * s2], c);
                const uint32_t a2 = nibble_pair<DT>(pa[2 * s2 + 1], c), a3 = nibble_pair<DT>(pb[2 * s2 + 1], c);
                const int k0 = 32 * w + 16 * s2 + 2 * c;
#pragma unroll
                for (int j = 0; j < QP_NT; j++) {
                    const uint16_t* xr = xs16 + (8 * j + g) * xld + k0;
                    const uint32_t b0 = *reinterpret_cast<const uint32_t*>(xr), b1 = *reinterpret_cast<const uint32_t*>(xr + 8);
                    mma16<DT>(d[j], a0, a1, a2, a3, b0, b1);
                }
            }
        }
        // the group's term: scale x (nibbles . x) + bias x (sum of x); rows g (elements 0, 1) and g + 8 (2, 3)
        const float sa0 = bf16_bits_to_float(sc0[grp]), sa1 = bf16_bits_to_float(sc0[8 * groups + grp]);
        const float sb0 = bf16_bits_to_float(bs0[grp]), sb1 = bf16_bits_to_float(bs0[8 * groups + grp]);
#pragma unroll
        for (int j = 0; j < QP_NT; j++) {
            const float2 xsv = *reinterpret_cast<const float2*>(xsum + grp * QP_TOKENS + 8 * j + 2 * c);
            acc[j][0] += fmaf(sb0, xsv.x, sa0 * d[j][0]);
            acc[j][1] += fmaf(sb0, xsv.y, sa0 * d[j][1]);
            acc[j][2] += fmaf(sb1, xsv.x, sa1 * d[j][2]);
            acc[j][3] += fmaf(sb1, xsv.y, sa1 * d[j][3]);
        }
    }
    __syncthreads();      // everyone is done with x: the head's outputs take its place, [tokens][128 rows] fp32
    float* y = reinterpret_cast<float*>(qp_smem);
#pragma unroll
    for (int j = 0; j < QP_NT; j++) {
        const int t = 8 * j + 2 * c, r = 16 * warp + g;
        y[t * HD + r] = Act<DT>::round(acc[j][0]);
        y[(t + 1) * HD + r] = Act<DT>::round(acc[j][1]);
        y[t * HD + r + 8] = Act<DT>::round(acc[j][2]);
        y[(t + 1) * HD + r + 8] = Act<DT>::round(acc[j][3]);
    }
    __syncthreads();

    // ---- epilogue: a warp a token, a lane holds dims lane + 32 i of the head
    for (int t = warp; t < ntok; t += QP_THREADS / 32) {
        const int b = tok0 + t;
        float v[4];
#pragma unroll
        for (int i = 0; i < 4; i++) v[i] = y[t * HD + lane + 32 * i];
        if (p.resid != nullptr) {
            // the o-projection's epilogues (gemv EPI 3 and 2): x = y or x += y, y rounded to the storage dtype, x in fp32
#pragma unroll
            for (int i = 0; i < 4; i++) {
                float* at = p.resid + size_t(b) * p.qkv_stride + size_t(head) * HD + lane + 32 * i;
                *at = p.resid_add ? *at + v[i] : v[i];
            }
            continue;
        }
        if (seg == 0) {
            // full layers: head norm with both gains; sliding layers: one gain, then RoPE at the token's position
            if (p.ng > 0) norm_rope_round<DT>(v, p.g1, p.g2, p.ng, p.ring_k ? p.seq_lens[b] - 1 : -1, p.rope_freq, lane);
#pragma unroll
            for (int i = 0; i < 4; i++) Act<DT>::store(p.qkv, size_t(b) * p.qkv_stride + size_t(head) * HD + lane + 32 * i, v[i]);
            continue;
        }
        if (p.ring_k != nullptr) {
            // the ring write of attn_sliding (attention.metal:47-62): k normed with its gain and rotated, v as it is
            const int pos = p.seq_lens[b] - 1;
            if (seg == 1 && p.kgain != nullptr) norm_rope_round<DT>(v, p.kgain, p.kgain, 1, pos, p.rope_freq, lane);
            uint8_t* dst = seg == 1 ? p.ring_k : p.ring_v;
            const size_t slot = size_t(b) * p.ring_stride + (size_t(seg_head) * p.ring + pos % p.ring) * HD;
#pragma unroll
            for (int i = 0; i < 4; i++) Act<DT>::store(dst, slot + lane + 32 * i, v[i]);
            continue;
        }
        if (p.pool == nullptr) {
#pragma unroll
            for (int i = 0; i < 4; i++) Act<DT>::store(p.qkv, size_t(b) * p.qkv_stride + size_t(head) * HD + lane + 32 * i, v[i]);
            continue;
        }
        // kv_append of this token's row (the k row normed first when the layer norms its keys), as kv_append_kernel does
        if (seg == 1 && p.norm_k) {
            float ss = 0.0f;
#pragma unroll
            for (int i = 0; i < 4; i++) ss = __fadd_rn(ss, __fmul_rn(v[i], v[i]));
            float tot = 0.0f;
            for (int l = 0; l < 32; l++) tot = __fadd_rn(tot, __shfl_sync(0xffffffffu, ss, l));
            const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, float(HD)), EPS32)));
#pragma unroll
            for (int i = 0; i < 4; i++) v[i] = __fmul_rn(v[i], r);
        }
        const int pos = p.seq_lens[b] - 1;
        const int block = p.block_table[size_t(b) * p.table_stride + pos / BLK];
        const int prow = pos % BLK;
        uint8_t* page = p.pool + ((size_t(block) * p.n_layers + p.layer) * p.n_kv_heads + seg_head) * p.page_bytes;
        int code[4];
        float scale;
        kv_row_quantise<DT>(v, code, scale);
        int8_t* codes = reinterpret_cast<int8_t*>(page) + (seg == 2 ? CODE_BYTES : 0) + prow * HD;
#pragma unroll
        for (int i = 0; i < 4; i++) codes[lane + 32 * i] = int8_t(code[i]);
        if (lane == 0) {
            uint8_t* sc = page + 2 * CODE_BYTES + (seg == 2 ? BLK * p.scale_bytes : 0);
            if (p.scale_bytes == 4) reinterpret_cast<float*>(sc)[prow] = scale;
            else reinterpret_cast<__half*>(sc)[prow] = __float2half_rn(scale);
        }
    }
}

}  // namespace embla

using namespace embla;

// x tile, sums of x, the head's scales and biases (bfloat16), the head's weight rows (padded)
static size_t qp_smem_bytes(int d_in) {
    return size_t(QP_TOKENS) * (d_in + 8) * 2 + size_t(d_in / 64) * QP_TOKENS * sizeof(float) + size_t(2) * HD * (d_in / 64) * 2 +
           size_t(HD) * (d_in / 2 + 16);
}

static EmblaStatus qkv_project_impl(EmblaAttn* ctx, const EmblaW4Matrix* wq, const EmblaW4Matrix* wk, const EmblaW4Matrix* wv,
                                    int32_t d_in, const void* x_dev, int64_t x_stride, int32_t batch, void* qkv_dev,
                                    int64_t qkv_stride, const EmblaQuery* gains, EmblaKVPool* pool, const EmblaKVView* view,
                                    int32_t norm_k, void* stream, const char* who, const EmblaRing* ring = nullptr,
                                    const int32_t* ring_seq_lens = nullptr, const void* kgain = nullptr) {
    if (!ctx || !wq || !wk || !wv || !x_dev || !qkv_dev) EMBLA_FAIL(EMBLA_BAD_ARG, "%s: null argument", who);
    EMBLA_CHECK_DEVICE(who, ctx, pool);
    const int Hq = ctx->cfg.n_q_heads, Hkv = ctx->cfg.n_kv_heads;
    if (d_in <= 0 || d_in % 64 || d_in > 2048) EMBLA_FAIL(EMBLA_BAD_ARG, "%s: d_in %d (a multiple of 64, at most 2048)", who, d_in);
    if (batch <= 0) EMBLA_FAIL(EMBLA_BAD_ARG, "%s: batch %d", who, batch);
    const EmblaW4Matrix* m[3] = {wq, wk, wv};
    const int want_rows[3] = {Hq * HD, Hkv * HD, Hkv * HD};
    QkvProjectParams p = {};
    for (int i = 0; i < 3; i++) {
        if (!m[i]->words_dev || !m[i]->scales_dev || !m[i]->biases_dev || m[i]->rows != want_rows[i])
            EMBLA_FAIL(EMBLA_BAD_ARG, "%s: matrix %d has %d rows (%d wanted) or a null part", who, i, m[i]->rows, want_rows[i]);
        if (reinterpret_cast<uintptr_t>(m[i]->words_dev) % 16) EMBLA_FAIL(EMBLA_BAD_ARG, "%s: matrix %d's words are not 16-byte aligned", who, i);
        p.w[i] = static_cast<const uint4*>(m[i]->words_dev);
        p.sc[i] = static_cast<const uint16_t*>(m[i]->scales_dev);
        p.bs[i] = static_cast<const uint16_t*>(m[i]->biases_dev);
    }
    if (qkv_stride < int64_t(Hq + 2 * Hkv) * HD) EMBLA_FAIL(EMBLA_BAD_ARG, "%s: qkv_stride %lld under the row's %d", who, (long long)qkv_stride, (Hq + 2 * Hkv) * HD);
    p.x = x_dev;
    p.qkv = qkv_dev;
    p.x_stride = x_stride;
    p.qkv_stride = qkv_stride;
    p.d_in = d_in;
    p.batch = batch;
    p.n_q_heads = Hq;
    p.n_kv_heads = Hkv;
    if (gains && !gains->prenormed) {
        if (gains->ng < 1 || gains->ng > 2 || !gains->g1_dev || (gains->ng == 2 && !gains->g2_dev))
            EMBLA_FAIL(EMBLA_BAD_ARG, "%s: ng %d without its gain vectors", who, gains->ng);
        p.ng = gains->ng;
        p.g1 = gains->g1_dev;
        p.g2 = gains->ng == 2 ? gains->g2_dev : gains->g1_dev;
    }
    if (pool) {
        if (!view || !view->block_table_dev || !view->seq_lens_dev || view->batch != batch)
            EMBLA_FAIL(EMBLA_BAD_ARG, "%s: the fused cache write needs a view of the same batch with a block table and sequence lengths", who);
        if (pool->kv_dtype != EMBLA_KV_INT8 || pool->n_kv_heads != Hkv || view->layer < 0 || view->layer >= pool->n_layers)
            EMBLA_FAIL(EMBLA_BAD_ARG, "%s: the pool must be the int8 pool of this context's kv heads, layer %d of %d", who, view->layer, pool->n_layers);
        p.pool = pool->base;
        p.block_table = view->block_table_dev;
        p.seq_lens = view->seq_lens_dev;
        p.table_stride = view->table_stride;
        p.layer = view->layer;
        p.n_layers = pool->n_layers;
        p.page_bytes = pool->page_bytes;
        p.scale_bytes = pool->scale_bytes;
        p.norm_k = norm_k;
    }
    if (x_stride % 8 || reinterpret_cast<uintptr_t>(x_dev) % 16)
        EMBLA_FAIL(EMBLA_BAD_ARG, "%s: x rows must start on 16 bytes (x_stride %lld a multiple of 8)", who, (long long)x_stride);
    if (ring) {
        if (!ring->k_dev || !ring->v_dev || !ring_seq_lens || ring->ring <= 0)
            EMBLA_FAIL(EMBLA_BAD_ARG, "%s: null ring or sequence lengths", who);
        if (p.ng > 1) EMBLA_FAIL(EMBLA_BAD_ARG, "%s: a sliding layer norms q with one gain vector", who);
        p.ring_k = static_cast<uint8_t*>(ring->k_dev);
        p.ring_v = static_cast<uint8_t*>(ring->v_dev);
        p.ring_stride = ring->seq_stride;
        p.ring = ring->ring;
        p.seq_lens = ring_seq_lens;
        p.kgain = kgain;
        fill_rope_freq(p.rope_freq);
    }
    p.ctl = kernel_ctl(ctx);
    const size_t smem = qp_smem_bytes(d_in);
    const bool bf = ctx->cfg.act_dtype == EMBLA_BF16;
    auto kern = bf ? qkv_project_kernel<EMBLA_BF16> : qkv_project_kernel<EMBLA_F16>;
    static bool configured[2][64] = {};
    if (!configured[bf][ctx->device & 63]) {
        EMBLA_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(qp_smem_bytes(2048))));
        configured[bf][ctx->device & 63] = true;
    }
    dim3 grid(Hq + 2 * Hkv, (batch + QP_TOKENS - 1) / QP_TOKENS);
    kern<<<grid, QP_THREADS, smem, static_cast<cudaStream_t>(stream)>>>(p);
    EMBLA_CUDA_TRY(cudaGetLastError());
    return EMBLA_OK;
}

extern "C" EmblaStatus embla_qkv_project(EmblaAttn* ctx, const EmblaW4Matrix* wq, const EmblaW4Matrix* wk, const EmblaW4Matrix* wv,
                                         int32_t d_in, const void* x_dev, int64_t x_stride, int32_t batch, void* qkv_dev,
                                         int64_t qkv_stride, void* stream) {
    return qkv_project_impl(ctx, wq, wk, wv, d_in, x_dev, x_stride, batch, qkv_dev, qkv_stride, nullptr, nullptr, nullptr, 0, stream,
                            "embla_qkv_project");
}

extern "C" EmblaStatus embla_qkv_project_full_step(EmblaAttn* ctx, const EmblaW4Matrix* wq, const EmblaW4Matrix* wk,
                                                   const EmblaW4Matrix* wv, int32_t d_in, const void* x_dev, int64_t x_stride,
                                                   const EmblaQuery* gains, EmblaKVPool* pool, const EmblaKVView* view,
                                                   int32_t norm_k, void* qkv_dev, int64_t qkv_stride, void* stream) {
    if (!pool || !view) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_qkv_project_full_step: null pool or view");
    return qkv_project_impl(ctx, wq, wk, wv, d_in, x_dev, x_stride, view->batch, qkv_dev, qkv_stride, gains, pool, view, norm_k, stream,
                            "embla_qkv_project_full_step");
}

extern "C" EmblaStatus embla_qkv_project_sliding_step(EmblaAttn* ctx, const EmblaW4Matrix* wq, const EmblaW4Matrix* wk,
                                                      const EmblaW4Matrix* wv, int32_t d_in, const void* x_dev, int64_t x_stride,
                                                      const void* qgain_dev, const void* kgain_dev, const EmblaRing* ring,
                                                      const int32_t* seq_lens_dev, int32_t batch, void* qkv_dev,
                                                      int64_t qkv_stride, void* stream) {
    if (!ring || !seq_lens_dev) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_qkv_project_sliding_step: null ring or sequence lengths");
    EmblaQuery gains = {};
    gains.prenormed = qgain_dev ? 0 : 1;
    gains.ng = qgain_dev ? 1 : 0;
    gains.g1_dev = qgain_dev;
    return qkv_project_impl(ctx, wq, wk, wv, d_in, x_dev, x_stride, batch, qkv_dev, qkv_stride, &gains, nullptr, nullptr, 0, stream,
                            "embla_qkv_project_sliding_step", ring, seq_lens_dev, kgain_dev);
}

// The consumer of the attention output: the o-projection (gemv with EPI 3 or 2, Engine.swift:830) from the rows
// embla_attn_*_decode wrote, into the fp32 residual stream.
extern "C" EmblaStatus embla_oproj(EmblaAttn* ctx, const EmblaW4Matrix* wo, int32_t d_in, const void* o_dev, int64_t o_stride,
                                   int32_t batch, float* x_dev, int64_t x_stride, int32_t accumulate, void* stream) {
    if (!ctx || !wo || !o_dev || !x_dev) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_oproj: null argument");
    EMBLA_CHECK_DEVICE("embla_oproj", ctx, static_cast<const EmblaKVPool*>(nullptr));
    if (d_in <= 0 || d_in % 64 || d_in > 2048) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_oproj: d_in %d (a multiple of 64, at most 2048)", d_in);
    if (batch <= 0 || !wo->words_dev || !wo->scales_dev || !wo->biases_dev || wo->rows <= 0 || wo->rows % HD)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_oproj: batch %d, rows %d (a multiple of 128)", batch, wo->rows);
    if (reinterpret_cast<uintptr_t>(wo->words_dev) % 16 || o_stride % 8 || reinterpret_cast<uintptr_t>(o_dev) % 16 || x_stride < wo->rows)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_oproj: words and input rows must start on 16 bytes, x_stride %lld must hold %d rows",
                   (long long)x_stride, wo->rows);
    QkvProjectParams p = {};
    p.w[0] = static_cast<const uint4*>(wo->words_dev);
    p.sc[0] = static_cast<const uint16_t*>(wo->scales_dev);
    p.bs[0] = static_cast<const uint16_t*>(wo->biases_dev);
    p.x = o_dev;
    p.x_stride = o_stride;
    p.qkv_stride = x_stride;
    p.resid = x_dev;
    p.resid_add = accumulate;
    p.d_in = d_in;
    p.batch = batch;
    p.n_q_heads = wo->rows / HD;     // every block of 128 rows is a "head" of the first matrix
    p.ctl = kernel_ctl(ctx);
    const size_t smem = qp_smem_bytes(d_in);
    const bool bf = ctx->cfg.act_dtype == EMBLA_BF16;
    auto kern = bf ? qkv_project_kernel<EMBLA_BF16> : qkv_project_kernel<EMBLA_F16>;
    EMBLA_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(qp_smem_bytes(2048))));
    dim3 grid(wo->rows / HD, (batch + QP_TOKENS - 1) / QP_TOKENS);
    kern<<<grid, QP_THREADS, smem, static_cast<cudaStream_t>(stream)>>>(p);
    EMBLA_CUDA_TRY(cudaGetLastError());
    return EMBLA_OK;
}

