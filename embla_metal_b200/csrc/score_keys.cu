// Key scoring of sparse layers that hold their own 16-bit keys: scores[kv head][j] = max over the
// kv head's query heads of q·k_j, the by-product the reference's full layers emit with SCORES
// (Sources/EmblaMetal/Kernels/attention.metal:146, 189, 203-205), as a pass of its own over the
// paged pool. The selection that follows compares index sets bit for bit, so every dot is ONE fp32
// fmaf chain over d = 0..127 (the order the CPU oracle fixes) — CUDA cores, not tensor cores.
//
// HBM-bound in bytes (256 B a key) but heavy in issue slots (G x 128 FMAs + 128 converts a key):
// a producer warp streams pages through a TMA ring (two 128-byte-wide swizzled boxes a page, dims
// 0-63 and 64-127); each consumer thread owns one key of the page and reads its row 16 bytes at a
// time, conflict-free under the swizzle; queries sit in shared memory as stored and are read as
// broadcast loads. The multiply-adds take the 16-bit operands directly (fma.rn.f32.f16 / .bf16).
#include "kv_row.cuh"

namespace embla {

constexpr int SK_CONSUMERS = 4;
constexpr int SK_THREADS = (SK_CONSUMERS + 1) * 32;
constexpr int SK_STAGE = BLK * HD * 2;   // K side of a 16-bit page
constexpr int SK_QLD = HD + 4;

struct ScoreParams {
    const int32_t* block_table;
    const int32_t* seq_lens;
    const void* q;
    float* scores;
    KernelCtl ctl;
    int64_t q_stride, scores_stride;
    int table_stride, layer, n_layers, n_kv_heads, rows_per_page, nsplit;
    // the current token's raw k and v rows, or NULL: appended to the 16-bit page by this launch (kv_append fused)
    uint8_t* pool;
    size_t page_bytes;
    const void* k_new;
    const void* v_new;
    int64_t kv_stride;
    int norm_k;
};

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

// acc = fma(q.lo, k.lo, acc); acc = fma(q.hi, k.hi, acc) on a packed pair of 16-bit values, the
// products exact and each step rounded once to fp32: the same result as converting to fp32 and
// calling fmaf, without the conversions (mixed-precision fma of sm_100).
template <int DT>
__device__ __forceinline__ void fma_pair(float& acc, uint32_t k, uint32_t q) {
    if (DT == EMBLA_F16) {
        asm("{\n .reg .b16 kl, kh, ql, qh;\n mov.b32 {kl, kh}, %1;\n mov.b32 {ql, qh}, %2;\n"
            " fma.rn.f32.f16 %0, ql, kl, %0;\n fma.rn.f32.f16 %0, qh, kh, %0;\n}\n"
            : "+f"(acc)
            : "r"(k), "r"(q));
    } else {
        asm("{\n .reg .b16 kl, kh, ql, qh;\n mov.b32 {kl, kh}, %1;\n mov.b32 {ql, qh}, %2;\n"
            " fma.rn.f32.bf16 %0, ql, kl, %0;\n fma.rn.f32.bf16 %0, qh, kh, %0;\n}\n"
            : "+f"(acc)
            : "r"(k), "r"(q));
    }
}

template <int DT, int G, int STAGES>
__global__ void __launch_bounds__(SK_THREADS) score_keys16_kernel(const __grid_constant__ CUtensorMap tmap,
                                                                 const ScoreParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* stages = smem;
    uint16_t* qs = reinterpret_cast<uint16_t*>(smem + STAGES * SK_STAGE);   // [G][128] in the activation dtype
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * SK_STAGE + G * SK_QLD * 4);
    uint64_t* empty = full + STAGES;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    trace_first(p.ctl.trace, 0);
    // An "early" launch (the kernel ahead of it in the stream writes none of this layer's pages) starts its first pages
    // before it waits for that kernel; seq_lens and the block table are inputs of the whole step.
    const int S = p.seq_lens[b];   // (an input of the whole step: read ahead of the wait, its latency hidden behind it)
    if (!p.ctl.early) {
        pdl_wait();
        pdl_launch_dependents();
    }
    const int npages = (S + BLK - 1) / BLK;
    const int pps = (npages + p.nsplit - 1) / p.nsplit;
    const int pg0 = split * pps;
    const int n = max(0, min(npages, pg0 + pps) - pg0);
    if (n == 0) {
        if (p.ctl.early) {
            pdl_wait();
            pdl_launch_dependents();
        }
        return;
    }
    // The CTA whose range ends with the sequence's last page also appends the current token (position S - 1): its
    // producer warp writes the k and v rows to the page for the kernels and steps to come and puts the k row into the
    // staged copy of the page, which may have been fetched before that write.
    const bool appends = p.k_new != nullptr && pg0 + n == npages;
    __shared__ uint64_t patched;
    __shared__ int s_failed, s_issued;

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
        uint8_t* dst = stages + st * SK_STAGE;
        mbar_expect_tx(&full[st], SK_STAGE);
        tma_load_2d(dst, &tmap, 0, int(page * p.rows_per_page), &full[st]);
        tma_load_2d(dst + BLK * 128, &tmap, 128, int(page * p.rows_per_page), &full[st]);
        *reinterpret_cast<volatile int*>(&s_issued) = i + 1;
        return true;
    };
    int next = 0;
    bool issuing = true;
    if (warp == SK_CONSUMERS) {
        // The producer warp starts before anyone else: lane i looks up the block of the range's page i (all lookups in
        // flight together), lane 0 sets the barriers up and requests the first pages into the stages (which start empty: no
        // wait), and in an early launch the lanes after those ask the L2 for the K sides of their pages: the HBM has little
        // else to do until the kernel ahead has finished.
        const int ahead = min(n, STAGES + (p.ctl.early ? min(p.ctl.l2_pages, 32 - STAGES) : 0));
        const int myblock = lane < ahead ? p.block_table[size_t(b) * p.table_stride + pg0 + lane] : 0;
        if (lane == 0) {
            for (int s = 0; s < STAGES; s++) {
                mbar_init(&full[s], 1);
                mbar_init(&empty[s], SK_CONSUMERS);
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
        if (lane >= STAGES && lane < ahead) {
            const size_t page = (size_t(myblock) * p.n_layers + p.layer) * p.n_kv_heads + kvh;
            l2_prefetch(p.pool + page * p.page_bytes, SK_STAGE);
        }
    }
    if (p.ctl.early) {
        pdl_wait();
        pdl_launch_dependents();
    }
    trace_first(p.ctl.trace, 1);
    for (int i = tid; i < G * HD; i += SK_THREADS)
        qs[i] = reinterpret_cast<const uint16_t*>(p.q)[size_t(b) * p.q_stride + size_t(kvh * G) * HD + i];
    __syncthreads();

    if (warp == SK_CONSUMERS) {
        float xk[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const int row = (S - 1) & (BLK - 1);
        if (appends) {
            // the whole warp, while the first pages are in flight: 16-bit pages take the rows rounded to the activation dtype
            const int block = p.block_table[size_t(b) * p.table_stride + npages - 1];
            uint8_t* page = p.pool + ((size_t(block) * p.n_layers + p.layer) * p.n_kv_heads + kvh) * p.page_bytes;
            const size_t off = size_t(b) * p.kv_stride + size_t(kvh) * HD;
            float xv[4];
            kv_row_load<DT>(p.k_new, off, p.norm_k != 0, lane, xk);
            kv_row_load<DT>(p.v_new, off, false, lane, xv);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                Act<DT>::store(page, size_t(row) * HD + lane + 32 * i, xk[i]);
                Act<DT>::store(page + BLK * HD * 2, size_t(row) * HD + lane + 32 * i, xv[i]);
            }
        }
        if (lane == 0)
            for (; next < n && issuing; next++) issuing = issue(next, -1);
        if (appends) {
            __syncwarp();
            const int il = n - 1;
            uint8_t* Kt = stages + (il % STAGES) * SK_STAGE;
            if (mbar_wait_bounded(p.ctl.wait_cycles, &full[il % STAGES], (il / STAGES) & 1)) {
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int d = lane + 32 * i;
                    Act<DT>::store(Kt + (d >> 6) * (BLK * 128) + row * 128 + ((((d & 63) >> 3) ^ (row & 7)) << 4) + (d & 7) * 2, 0, xk[i]);
                }
            } else if (lane == 0) {
                atomicExch(p.ctl.err, ERR_WAIT_FULL);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&patched);
        }
    }
    if (warp < SK_CONSUMERS) {
        const int r = warp * 32 + lane;   // this thread's key of every page
        for (int i = 0; i < n; i++) {
            const int st = i % STAGES, use = i / STAGES;
            // (the decision is the warp's: a warp that leaves the loop leaves it whole)
            if (!__all_sync(0xffffffffu, mbar_wait_bounded(p.ctl.wait_cycles, &full[st], use & 1) &&
                                             (!(appends && i == n - 1) || mbar_wait_bounded(p.ctl.wait_cycles, &patched, 0)))) {
                atomicExch(p.ctl.err, ERR_WAIT_FULL);
                *reinterpret_cast<volatile int*>(&s_failed) = 1;
                break;
            }
            const uint32_t Kb = smem_u32(stages + st * SK_STAGE) + r * 128, qa = smem_u32(qs);
            float dot[G];
#pragma unroll
            for (int h = 0; h < G; h++) dot[h] = 0.0f;
#pragma unroll
            for (int half = 0; half < 2; half++) {
#pragma unroll
                for (int ch = 0; ch < 8; ch++) {
                    const uint4 kw = lds128(Kb + half * (BLK * 128) + ((ch ^ (r & 7)) << 4));
                    const int d = half * 64 + ch * 8;
#pragma unroll
                    for (int h = 0; h < G; h++) {
                        const uint4 qw = lds128(qa + (h * HD + d) * 2);   // one address a warp: a broadcast
                        fma_pair<DT>(dot[h], kw.x, qw.x);
                        fma_pair<DT>(dot[h], kw.y, qw.y);
                        fma_pair<DT>(dot[h], kw.z, qw.z);
                        fma_pair<DT>(dot[h], kw.w, qw.w);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[st]);
            float best = dot[0];
#pragma unroll
            for (int h = 1; h < G; h++)
                if (dot[h] > best) best = dot[h];
            const int key = (pg0 + i) * BLK + r;
            if (key < S) p.scores[(size_t(b) * p.n_kv_heads + kvh) * p.scores_stride + key] = best;
        }
    }
    trace_last(p.ctl.trace, 2);
    // A wait that gave up: no thread leaves while a copy may still be on its way into this CTA's stages.
    __syncthreads();
    if (s_failed && tid == 0) {
        for (int i = max(0, s_issued - STAGES); i < s_issued; i++)
            if (!mbar_wait_bounded(p.ctl.wait_cycles, &full[i % STAGES], (i / STAGES) & 1)) atomicExch(p.ctl.err, ERR_WAIT_DRAIN);
    }
    trace_last(p.ctl.trace, 3);
}

int choose_splits(int pairs, int pages, int slots, int max_slots);

template <int DT, int G>
static EmblaStatus launch_score(EmblaAttn* ctx, const EmblaKVPool* pool, const ScoreParams& p, int batch, cudaStream_t s) {
    constexpr int STAGES = 3;
    constexpr size_t smem = 1024 + STAGES * SK_STAGE + G * SK_QLD * 4 + 2 * STAGES * 8;
    auto kern = score_keys16_kernel<DT, G, STAGES>;
    static bool configured[64] = {};
    if (!configured[ctx->device & 63]) {
        EMBLA_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        configured[ctx->device & 63] = true;
    }
    dim3 grid(p.nsplit, p.n_kv_heads, batch);
    EMBLA_CUDA_TRY(launch_kernel(ctx->pdl, kern, grid, dim3(SK_THREADS), smem, s, pool->tmap_codes, p));
    EMBLA_CUDA_TRY(cudaGetLastError());
    return EMBLA_OK;
}

}  // namespace embla

using namespace embla;

static EmblaStatus score_keys_impl(EmblaAttn* ctx, const EmblaKVPool* pool, const EmblaKVView* view, const void* q_dev,
                                   int64_t q_stride, float* scores_dev, int64_t scores_stride, const void* k_new,
                                   const void* v_new, int64_t kv_stride, int32_t norm_k, void* stream) {
    if (!ctx || !pool || !view || !q_dev || !scores_dev) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_score_keys: null argument");
    EMBLA_CHECK_DEVICE("embla_score_keys", ctx, pool);
    if (pool->kv_dtype != EMBLA_KV_16BIT) EMBLA_FAIL(EMBLA_UNSUPPORTED, "embla_score_keys: the pool is not 16-bit");
    if (pool->n_kv_heads != ctx->cfg.n_kv_heads || view->layer < 0 || view->layer >= pool->n_layers)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_score_keys: pool/layer mismatch");
    if (view->batch <= 0 || view->batch > ctx->cfg.max_batch || !view->block_table_dev || !view->seq_lens_dev)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_score_keys: bad view (batch %d)", view->batch);
    const int max_len = view->max_seq_len > 0 ? view->max_seq_len : ctx->cfg.max_context;
    if (scores_stride < max_len)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_score_keys: scores_stride %lld under max_seq_len %d", (long long)scores_stride, max_len);
    ScoreParams p = {};
    p.block_table = view->block_table_dev;
    p.seq_lens = view->seq_lens_dev;
    p.q = q_dev;
    p.scores = scores_dev;
    p.ctl = kernel_ctl(ctx);
    p.q_stride = q_stride;
    p.scores_stride = scores_stride;
    p.table_stride = view->table_stride;
    p.layer = view->layer;
    p.n_layers = pool->n_layers;
    p.n_kv_heads = pool->n_kv_heads;
    p.rows_per_page = pool->rows_per_page;
    p.pool = pool->base;
    p.page_bytes = pool->page_bytes;
    p.k_new = k_new;
    p.v_new = v_new;
    p.kv_stride = kv_stride;
    p.norm_k = norm_k;
    const int pages = (max_len + BLK - 1) / BLK;
    p.nsplit = choose_splits(view->batch * pool->n_kv_heads, pages, 2 * ctx->sm_count, 1 << 30);
    const int G = ctx->cfg.n_q_heads / ctx->cfg.n_kv_heads;
    const bool bf = ctx->cfg.act_dtype == EMBLA_BF16;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
#define EMBLA_SK(G_) (bf ? launch_score<EMBLA_BF16, G_>(ctx, pool, p, view->batch, s) : launch_score<EMBLA_F16, G_>(ctx, pool, p, view->batch, s))
    switch (G) {
        case 1: return EMBLA_SK(1);
        case 2: return EMBLA_SK(2);
        case 4: return EMBLA_SK(4);
        case 8: return EMBLA_SK(8);
        default: EMBLA_FAIL(EMBLA_UNSUPPORTED, "embla_score_keys: %d query heads per kv head (1, 2, 4 or 8)", G);
    }
#undef EMBLA_SK
}

extern "C" EmblaStatus embla_score_keys(EmblaAttn* ctx, const EmblaKVPool* pool, const EmblaKVView* view,
                                        const void* q_dev, int64_t q_stride, float* scores_dev, int64_t scores_stride,
                                        void* stream) {
    return score_keys_impl(ctx, pool, view, q_dev, q_stride, scores_dev, scores_stride, nullptr, nullptr, 0, 0, stream);
}

extern "C" EmblaStatus embla_score_keys_step(EmblaAttn* ctx, EmblaKVPool* pool, const EmblaKVView* view, const void* q_dev,
                                             int64_t q_stride, const void* k_dev, const void* v_dev, int64_t kv_stride,
                                             int32_t norm_k, float* scores_dev, int64_t scores_stride, void* stream) {
    if (!k_dev || !v_dev) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_score_keys_step: null k or v");
    return score_keys_impl(ctx, pool, view, q_dev, q_stride, scores_dev, scores_stride, k_dev, v_dev, kv_stride, norm_k, stream);
}
