// Prefill-chunk attention of the full layers: causal ReLU² of up to 2048 new tokens over the int8
// paged cache (their own keys already appended). Replaces relu2_prefill_nax
// (Sources/EmblaMetal/Kernels/attn_nax.metal:61-364) with q_prep_b
// (Sources/EmblaMetal/Kernels/prefill.metal:408-426); dispatch Sources/EmblaMetal/Prefill.swift:378-407.
//
// This is the one dense contraction of the path, so it runs on the 5th-generation tensor cores:
//   S = Q Kᵀ   tcgen05.mma kind::f16, M = 128 queries, N = 128 keys (one page), K = 128 dims, fp32 in TMEM
//   O += P V   tcgen05.mma kind::f16, A = P read straight from TMEM, B = V from shared memory (MN-major)
// One CTA owns 256 consecutive tokens of one query head as two tiles of 128 and walks the sequence's pages;
// both tiles use every converted page, which halves the conversion work per MMA (with fewer such units than SMs a unit's
// pages are shared among CTAs: launch_prefill chooses how, and how their partial sums meet):
//   warp 12     TMA producer: one side (K or V: 128 int8 code rows, swizzled box) at a time into a 3-slot ring,
//               the page's scales with its K side
//   warps 8-11  converters: int8 codes -> fp16 (exact), times the row's factor (kscale/√D or vscale), into the
//               UMMA operand layout [dims 0-63 | 64-127][128 keys][128 B], 128-byte swizzle — the same layout
//               serves K as the K-major B operand of Q Kᵀ and V as the MN-major B operand of P V; 3 buffers
//   warp 13     MMA issuer (one thread), per page: S0(j), P V1(j-1), S1(j), P V0(j) — while the ReLU² warps of
//               one tile work on its scores the tensor pipe runs the other tile's products
//   warps 0-7   two warpgroups, one per tile, one query row a thread: tcgen05.ld S, p = max(s,0)² masked
//               causally, row sums in fp32, P as fp16 back into TMEM over the consumed S columns
//               (tcgen05.st); at the end O / (√D + Σp)
// TMEM (512 columns): per tile S 128 (P aliases its first 64) and O 128. q is converted to fp16 once (bf16 values are exact
// in fp16 inside its normal range); int8 codes and their products are exact; accumulation is fp32.
// Every wait is bounded; a wait that runs out sets the context's error word and the CTA winds down.
#include "kv_row.cuh"
#include "tc05.cuh"

namespace embla {

constexpr int PF_CONV_WARPS = 4;                          // converter warps (8 measured no faster)
constexpr int PF_PRODUCER = 8 + PF_CONV_WARPS;            // warp roles: 0-7 ReLU², 8.. converters, then TMA producer, MMA issuer
constexpr int PF_MMA = PF_PRODUCER + 1;
constexpr int PF_THREADS = (PF_MMA + 1) * 32;
constexpr int PF_TILE16 = BLK * HD * 2;            // 32 KiB: 128 rows x 128 dims fp16
constexpr int PF_KVBUFS = 3;
constexpr int PF_MAX_PEERS = 8;
constexpr int PF_BAL_UNITS = 256, PF_BAL_PIECES = 512;    // most units and pieces (CTAs) of a balanced launch
// The queries enter the tensor cores scaled by 2^-3 (exact), so the weights p = relu(s)^2, which the kernel keeps as
// fp16 (P in TMEM, packed row sums), come out scaled by 2^-6: a score of 2047 still squares inside fp16's range (the
// reference keeps P in fp32, attn_nax.metal:11), and fp16's gradual underflow keeps the small weights to 2^-24 of the
// scaled unit. The sink of the denominator takes the same factor, so O / (sink + sum p) is unchanged.
constexpr float PF_QSCALE = 0.125f, PF_PSCALE = PF_QSCALE * PF_QSCALE;
// QK8: the integer dots are bounded by 127 x 127 x 128 whatever the queries' size, so the ReLU² warps scale them by the
// key's factor and this constant only, u = S x kscale / sqrt(D) x 2^-8 (u^2 stays inside fp16 for key scales up to 0.25);
// the row's own factor rho = qscale x PF_QSCALE x 2^8 multiplies every weight of the row by rho^2, so it only moves the
// sink: O / (sink + sum p) = sum u^2 v / (sink / rho^2 + sum u^2).
constexpr float PF_QK8_C0 = 1.0f / 256.0f;
// alignment slack, 2 Q tiles, 3 converted sides, 3 raw int8 sides, 2 pages' scales, barriers
constexpr size_t PF_SMEM = 1024 + 2 * PF_TILE16 + PF_KVBUFS * PF_TILE16 + PF_KVBUFS * CODE_BYTES + 2 * 1024 + 256 + 2 * 1024;

struct PfPiece;
struct PrefillParams {
    const uint8_t* pool;
    const int32_t* block_table;
    const int32_t* pos0;       // [batch] position of the chunk's first token
    const void* q;
    const void* g1;
    const void* g2;
    void* o;
    // scatter mode (head-sharded prefill on several GPUs): the output rows also go, with plain stores, to these addresses in
    // other GPUs' memory (each where this rank's slab starts inside that GPU's token-major output, same strides)
    void* o_peer[PF_MAX_PEERS];
    int n_peers;
    KernelCtl ctl;
    float* partials;      // split-KV: [unit][split][tile][128 + 1 columns][128 rows] fp32 (unnormalised O, then the row sums)
    int* counters;        // [2][units]: the unit's ranges that have announced themselves, and those whose partials are written
    int64_t q_token_stride, q_seq_stride, o_token_stride, o_seq_stride;
    size_t page_bytes;
    int table_stride, layer, n_layers, n_kv_heads, G, scale_bytes, rows_per_page, n_tokens, prenormed, nsplit;
    int cls;              // cluster size (0: none, else = nsplit): the page ranges of a unit are the CTAs of one thread-block
                          // cluster, whose partial sums stay in shared memory
    int heads, pairs;     // query heads and 256-token tile pairs of the launch: unit = (sequence x heads + head) x pairs + pair
    int units;            // sequences x heads x pairs
    int balanced;         // balanced launch (prefill_pieces_kernel): CTA k takes pieces[k]
    const struct PfPiece* pieces;
    int reduce_later;     // every range leaves its partial in the scratch and prefill_reduce_kernel adds them (units cut into
                          // more ranges than one CTA should add up alone)
    int2* unit_slots;     // [unit] (first slot, ranges) for that kernel
};

// One side (K or V) of a raw int8 page -> fp16 in the UMMA layout. 128 converter threads; lanes of a
// quarter warp take 8 consecutive rows of one 16-byte chunk, so reads and writes are conflict-free.
__device__ __forceinline__ uint32_t h2_scaled(uint32_t x, uint32_t sel, __half2 sc) {
    const uint32_t v = h2_from_biased_bytes(x, sel);
    const __half2 r = __hmul2(*reinterpret_cast<const __half2*>(&v), sc);
    return *reinterpret_cast<const uint32_t*>(&r);
}

// `scales[row] * mult`: the row's dequantisation factor (keys: kscale / sqrt(D); values: vscale), applied as
// fp16 after the exact widening, so the ReLU² warps need no per-key factors.
template <int SB>
__device__ __forceinline__ void convert_side(const uint8_t* raw, uint8_t* dst, int ctid, const uint8_t* scales, float mult) {
    constexpr int RG = PF_CONV_WARPS / 2;   // groups of 8 rows the converter threads cover at once
    const int rl = ctid & 7, ch = (ctid >> 3) & 7, rg = ctid >> 6;
#pragma unroll
    for (int it = 0; it < BLK / (8 * RG); it++) {
        const int row = it * 8 * RG + rg * 8 + rl;
        const uint4 w = *reinterpret_cast<const uint4*>(raw + row * 128 + ((ch ^ (row & 7)) << 4));
        const float f = SB == 4 ? reinterpret_cast<const float*>(scales)[row] : __half2float(reinterpret_cast<const __half*>(scales)[row]);
        const __half2 sc = __float2half2_rn(f * mult);
        const uint32_t x[4] = {w.x ^ 0x80808080u, w.y ^ 0x80808080u, w.z ^ 0x80808080u, w.w ^ 0x80808080u};
        uint4 lo, hi;   // dims 16ch..16ch+7 and 16ch+8..16ch+15
        lo.x = h2_scaled(x[0], 0x4140, sc);
        lo.y = h2_scaled(x[0], 0x4342, sc);
        lo.z = h2_scaled(x[1], 0x4140, sc);
        lo.w = h2_scaled(x[1], 0x4342, sc);
        hi.x = h2_scaled(x[2], 0x4140, sc);
        hi.y = h2_scaled(x[2], 0x4342, sc);
        hi.z = h2_scaled(x[3], 0x4140, sc);
        hi.w = h2_scaled(x[3], 0x4342, sc);
        uint8_t* base = dst + (ch >> 2) * (BLK * 128) + row * 128;
        const int c16 = (2 * ch) & 7;
        *reinterpret_cast<uint4*>(base + ((c16 ^ (row & 7)) << 4)) = lo;
        *reinterpret_cast<uint4*>(base + (((c16 + 1) ^ (row & 7)) << 4)) = hi;
    }
}

// QK8: the reference's int8 Q Kᵀ variant (attn_nax.metal:14-22, 124-204 with q_prep_b's QK8 branch, prefill.metal:421-422;
// switched on by EMBLA_ATT8, Prefill.swift:142-144): every query row is quantised like a cache row (write_row8: rounded to
// the activation dtype, codes rint(x 127 / max|x|), scale max|x| / 127), S = Q8 K8ᵀ runs as tcgen05.mma kind::i8 on the
// cache's codes as they are (int32 in TMEM, exact), and the ReLU² warps scale it: s = S x qscale(row) x kscale(key) / √D.
// P V stays fp16 as in the other variant. Twice the tensor rate for Q Kᵀ, and no conversion of the K side at all.
// the barrier of the eight ReLU² warps among themselves (the other warps are in their own loops or done)
__device__ __forceinline__ void relu_warps_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// A CTA's work: a page range [jb, je) of one unit (two query tiles of one head), as the kernel at the end of this file
// works it out from the block index.
struct PfSegment {
    int h, b, pair_ix;      // head, sequence, tile pair of the unit
    int split, nparts;      // which of the unit's page ranges this is, of how many
    int slot0;              // the unit's first slot in the scratch
    int jb, je;             // the pages
};

template <int DT, int SB, bool QK8>
__device__ __forceinline__ void full_prefill_segment(const CUtensorMap& tmap, const PrefillParams& p, const PfSegment sg) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* Qs = smem;                                               // [2 tiles][32 KiB]
    uint8_t* kvb = smem + 2 * PF_TILE16;                              // [3][32 KiB] converted K / V sides
    uint8_t* raw = kvb + PF_KVBUFS * PF_TILE16;                       // [3][16 KiB] int8 sides as loaded
    uint8_t* scl = raw + PF_KVBUFS * CODE_BYTES;                      // [2 pages][K scales | V scales], 1 KiB each
    uint64_t* bars = reinterpret_cast<uint64_t*>(scl + 2 * 1024);
    float* qsc = reinterpret_cast<float*>(scl + 2 * 1024 + 256);     // QK8: [2 tiles][128] 1 / rho^2 of the int8 query rows
    float* kfac = qsc + 2 * BLK;                                      // QK8: [2 pages][128] kscale / sqrt(D) x 2^-8 of the page's keys
    uint64_t* raw_full = bars;            // [3]
    uint64_t* raw_empty = bars + 3;       // [3]
    uint64_t* kv_ready = bars + 6;        // [3]
    uint64_t* kv_free = bars + 9;         // [3]
    uint64_t* s_full = bars + 12;         // [2 tiles]
    uint64_t* p_ready = bars + 14;        // [2 tiles]
    uint64_t* o_done = bars + 16;
    uint64_t* kf_ready = bars + 17;       // [2 pages] QK8: the page's key factors are set out (converters -> ReLU² warps)
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort, s_last;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = sg.h, b = sg.b, pair_ix = sg.pair_ix, split = sg.split, nparts = sg.nparts, slot0 = sg.slot0;
    const int jb = sg.jb, je = sg.je;
    const int unit = (b * p.heads + h) * p.pairs + pair_ix;
    const int kvh = h / p.G;
    const int p0 = p.pos0[b];
    // two query tiles of 128 consecutive tokens each share every converted page
    int t0[2], rows[2], npg[2];
#pragma unroll
    for (int x = 0; x < 2; x++) {
        t0[x] = (2 * pair_ix + x) * BLK;
        rows[x] = max(0, min(BLK, p.n_tokens - t0[x]));
        npg[x] = rows[x] > 0 ? (p0 + t0[x] + rows[x] - 1) / BLK + 1 : 0;
    }
    const int n = max(0, je - jb);
    // The producer lane sets the barriers up and requests the first pages while the other warps stage the query tiles.
    if (warp == PF_PRODUCER && lane == 0) {
        for (int i = 0; i < 3; i++) {
            mbar_init(&raw_full[i], 1);
            mbar_init(&raw_empty[i], PF_CONV_WARPS);
            mbar_init(&kv_ready[i], PF_CONV_WARPS);
            mbar_init(&kv_free[i], 1);
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(&s_full[i], 1);
            mbar_init(&p_ready[i], 4);
        }
        mbar_init(o_done, 1);
        mbar_init(&kf_ready[0], PF_CONV_WARPS);
        mbar_init(&kf_ready[1], PF_CONV_WARPS);
        s_abort = 0;
        fence_barrier_init();
    }
    // conversion c = 2 j + side takes ring slot c % 3; page j's scales go to scl[j & 1]
    auto request = [&](int c) {
        const int j = jb + (c >> 1), side = c & 1, slot = c % 3;
        const int block = p.block_table[size_t(b) * p.table_stride + j];
        const long page = (long(block) * p.n_layers + p.layer) * p.n_kv_heads + kvh;
        mbar_expect_tx(&raw_full[slot], CODE_BYTES + (side == 0 ? 2 * BLK * SB : 0));
        tma_load_2d(raw + slot * CODE_BYTES, &tmap, 0, int(page * p.rows_per_page) + side * BLK, &raw_full[slot]);
        if (side == 0)
            bulk_load_1d(scl + ((c >> 1) & 1) * 1024, p.pool + size_t(page) * p.page_bytes + 2 * CODE_BYTES, 2 * BLK * SB, &raw_full[slot]);
    };
    int requested = 0;        // (producer lane) conversions requested so far
    if (warp == PF_PRODUCER && lane == 0)
        for (; requested < min(3, 2 * n) && requested != p.ctl.stall_at; requested++) request(requested);
    if (warp == PF_MMA) tmem_alloc(&s_tmem, 512);
    // the staging warps: every warp but the producer
    constexpr int SW = PF_THREADS / 32 - 1;
    const int swarp = warp < PF_PRODUCER ? warp : warp - 1, stid = swarp * 32 + lane;

    // ---- Q tiles: [128 tokens][128 dims] of head h as fp16 in the K-major swizzled layout
    if (!QK8 && p.prenormed && warp != PF_PRODUCER) {
        // rows as they are, times the query scale: 16 bytes a thread and trip, every load of a thread (both tiles) in flight
        // before the first store
        constexpr int TRIPS = (BLK * 16 + SW * 32 - 1) / (SW * 32);
        uint4 v[2][TRIPS];
#pragma unroll
        for (int x = 0; x < 2; x++)
#pragma unroll
            for (int k = 0; k < TRIPS; k++) {
                const int i = stid + k * (SW * 32), r = i >> 4, c8 = i & 15;
                v[x][k] = make_uint4(0, 0, 0, 0);
                if (i < BLK * 16 && r < rows[x]) {
                    const size_t off = size_t(b) * p.q_seq_stride + size_t(t0[x] + r) * p.q_token_stride + size_t(h) * HD + c8 * 8;
                    v[x][k] = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.q) + off);
                }
            }
#pragma unroll
        for (int x = 0; x < 2; x++)
#pragma unroll
            for (int k = 0; k < TRIPS; k++) {
                const int i = stid + k * (SW * 32), r = i >> 4, c8 = i & 15;
                if (i >= BLK * 16) continue;
                uint32_t* w = &v[x][k].x;
                if (DT == EMBLA_BF16) {
#pragma unroll
                    for (int e = 0; e < 4; e++)
                        w[e] = pack_h2(__uint_as_float(w[e] << 16) * PF_QSCALE, __uint_as_float(w[e] & 0xffff0000u) * PF_QSCALE);
                } else {
                    const __half2 qs2 = __float2half2_rn(PF_QSCALE);
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const __half2 t = __hmul2(*reinterpret_cast<const __half2*>(&w[e]), qs2);
                        w[e] = *reinterpret_cast<const uint32_t*>(&t);
                    }
                }
                *reinterpret_cast<uint4*>(Qs + x * PF_TILE16 + (c8 >> 3) * (BLK * 128) + r * 128 + (((c8 & 7) ^ (r & 7)) << 4)) = v[x][k];
            }
    }
    for (int x = 0; x < 2 && warp != PF_PRODUCER && (QK8 || !p.prenormed); x++) {
        uint8_t* Qx = Qs + x * PF_TILE16;
        if (QK8) {
            // one warp a row, four rows a trip with their loads in flight together: head norm (unless the rows come normed),
            // then the row as int8 codes, K-major [128 rows][128 B] under the 128-byte swizzle, and its scale
            for (int r4 = swarp * 4; r4 < BLK; r4 += 4 * SW) {
                float xq[4][4];
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const int r = r4 + k;
                    const size_t off = size_t(b) * p.q_seq_stride + size_t(t0[x] + r) * p.q_token_stride + size_t(h) * HD;
#pragma unroll
                    for (int i = 0; i < 4; i++) xq[k][i] = r < rows[x] ? Act<DT>::load(p.q, off + lane + 32 * i) : 0.0f;
                }
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const int r = r4 + k;
                    if (r < rows[x] && !p.prenormed) {
                        float ss = 0.0f;
#pragma unroll
                        for (int i = 0; i < 4; i++) ss = __fadd_rn(ss, __fmul_rn(xq[k][i], xq[k][i]));
                        float tot = 0.0f;
                        for (int l = 0; l < 32; l++) tot = __fadd_rn(tot, __shfl_sync(0xffffffffu, ss, l));
                        const float rr = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, float(HD)), EPS32)));
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const int d = lane + 32 * i;
                            float gn = __fmul_rn(rr, __fadd_rn(1.0f, Act<DT>::load(p.g1, d)));
                            gn = __fmul_rn(gn, __fadd_rn(1.0f, Act<DT>::load(p.g2, d)));
                            xq[k][i] = __fmul_rn(xq[k][i], gn);
                        }
                    }
                    int code[4];
                    float qscale;
                    kv_row_quantise<DT>(xq[k], code, qscale);   // (rows past the chunk: zeros, scale 0)
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const int d = lane + 32 * i;
                        Qx[r * 128 + (((d >> 4) ^ (r & 7)) << 4) + (d & 15)] = uint8_t(int8_t(code[i]));
                    }
                    if (lane == 0) {
                        const float rho = qscale * PF_QSCALE / PF_QK8_C0;
                        qsc[x * BLK + r] = 1.0f / (rho * rho);   // (a zero row: infinity, and its output 0 / infinity = 0)
                    }
                }
            }
        } else {
            // q_prep_b: head norm with both gains in the oracle's operation order, rounded to the activation dtype; four
            // rows a warp and trip, their loads in flight together before the norms
            for (int r4 = swarp * 4; r4 < BLK; r4 += 4 * SW) {
                float xq[4][4];
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const int r = r4 + k;
                    const size_t off = size_t(b) * p.q_seq_stride + size_t(t0[x] + r) * p.q_token_stride + size_t(h) * HD;
#pragma unroll
                    for (int i = 0; i < 4; i++) xq[k][i] = r < rows[x] ? Act<DT>::load(p.q, off + lane + 32 * i) : 0.0f;
                }
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const int r = r4 + k;
                    if (r < rows[x]) {
                        float ss = 0.0f;
#pragma unroll
                        for (int i = 0; i < 4; i++) ss = __fadd_rn(ss, __fmul_rn(xq[k][i], xq[k][i]));
                        float tot = 0.0f;
                        for (int l = 0; l < 32; l++) tot = __fadd_rn(tot, __shfl_sync(0xffffffffu, ss, l));
                        const float rr = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, float(HD)), EPS32)));
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const int d = lane + 32 * i;
                            float gn = __fmul_rn(rr, __fadd_rn(1.0f, Act<DT>::load(p.g1, d)));
                            gn = __fmul_rn(gn, __fadd_rn(1.0f, Act<DT>::load(p.g2, d)));
                            xq[k][i] = Act<DT>::round(__fmul_rn(xq[k][i], gn));
                        }
                    }
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const int d = lane + 32 * i, c8 = d >> 3;
                        *reinterpret_cast<__half*>(Qx + (c8 >> 3) * (BLK * 128) + r * 128 + (((c8 & 7) ^ (r & 7)) << 4) + (d & 7) * 2) =
                            __float2half_rn(xq[k][i] * PF_QSCALE);
                    }
                }
            }
        }
    }
    fence_proxy_async();      // Q was written by ordinary stores; the tensor pipe reads it through the async proxy
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    // TMEM columns: S/P of tile 0 at 0, of tile 1 at 128 (P overwrites the first 64 columns of its S); O at 256, 384

    if (warp == PF_PRODUCER) {
        // ---- TMA producer: the conversions after the first three, each once its ring slot is free
        if (lane == 0) {
            for (int c = requested; c < 2 * n; c++) {
                const int slot = c % 3;
                if (c == p.ctl.stall_at) break;   // diagnostic stall: the converters' wait for this side runs out
                if (c >= 3 && !mbar_wait_bounded(p.ctl.wait_cycles, &raw_empty[slot], ((c / 3) - 1) & 1)) {
                    atomicExch(p.ctl.err, ERR_WAIT_EMPTY);
                    break;
                }
                if (*reinterpret_cast<volatile int*>(&s_abort)) break;
                request(c);
            }
        }
    } else if (warp == PF_MMA) {
        // ---- MMA issuer. Per page: S0(j), PV1(j-1), S1(j), PV0(j): while the ReLU² warps of one tile work on its
        // scores, the tensor pipe runs the other tile's products. All MMAs of one thread execute in issue order,
        // which is what lets P overwrite S and S(j+1) overwrite P(j).
        if (lane == 0) {
            const uint32_t qa = smem_u32(Qs);
            bool ok = true;
            // i = page index inside this CTA's range (buffers and barrier phases count from 0), jb + i = the page
            auto issue_s = [&](int x, int i) {
                const uint32_t ka = smem_u32(kvb + ((2 * i) % 3) * PF_TILE16);
                if (QK8) {
                    // int8 operands: one [128 rows][128 B] tile holds all 128 dims, 32 of them (32 bytes) an instruction
#pragma unroll
                    for (int ks = 0; ks < 4; ks++)
                        umma_ss_i8(tmem + 128 * x, umma_desc(qa + x * PF_TILE16 + ks * 32, 16, 1024), umma_desc(ka + ks * 32, 16, 1024),
                                   PF_IDESC_QK8, ks > 0);
                } else {
#pragma unroll
                    for (int ks = 0; ks < 8; ks++) {
                        const uint32_t koff = (ks >> 2) * (BLK * 128) + (ks & 3) * 32;
                        umma_ss(tmem + 128 * x, umma_desc(qa + x * PF_TILE16 + koff, 16, 1024), umma_desc(ka + koff, 16, 1024), PF_IDESC_QK, ks > 0);
                    }
                }
                tc_commit(&s_full[x]);
            };
            auto issue_pv = [&](int x, int i) {
                const uint32_t va = smem_u32(kvb + ((2 * i + 1) % 3) * PF_TILE16);
#pragma unroll
                for (int ks = 0; ks < 8; ks++)
                    umma_ts(tmem + 256 + 128 * x, tmem + 128 * x + 8 * ks, umma_desc(va + ks * 2048, BLK * 128, 1024), PF_IDESC_PV,
                            (i > 0) | (ks > 0));
            };
            for (int i = 0; i <= n && ok; i++) {
                const bool a0 = i < n && jb + i < npg[0], a1 = i < n && jb + i < npg[1];   // tiles active on this page
                const bool b1 = i >= 1 && jb + i - 1 < npg[1];                              // tile 1 had the page before
                if (a0 || a1) {
                    ok = mbar_wait_bounded(p.ctl.wait_cycles, &kv_ready[(2 * i) % 3], ((2 * i) / 3) & 1);
                    if (!ok) break;
                    tc_fence_after();
                }
                if (a0) issue_s(0, i);
                if (b1) {
                    const int cv = 2 * (i - 1) + 1;
                    ok = mbar_wait_bounded(p.ctl.wait_cycles, &p_ready[1], (i - 1) & 1) && mbar_wait_bounded(p.ctl.wait_cycles, &kv_ready[cv % 3], (cv / 3) & 1);
                    if (!ok) break;
                    tc_fence_after();
                    issue_pv(1, i - 1);
                }
                if (i >= 1) tc_commit(&kv_free[(2 * (i - 1) + 1) % 3]);   // V of the page before: both tiles' P V are issued
                if (a1) issue_s(1, i);
                if (a0 || a1) tc_commit(&kv_free[(2 * i) % 3]);           // K of this page
                if (a0) {
                    const int cv = 2 * i + 1;
                    ok = mbar_wait_bounded(p.ctl.wait_cycles, &p_ready[0], i & 1) && mbar_wait_bounded(p.ctl.wait_cycles, &kv_ready[cv % 3], (cv / 3) & 1);
                    if (!ok) break;
                    tc_fence_after();
                    issue_pv(0, i);
                }
            }
            if (!ok) {
                atomicExch(p.ctl.err, ERR_WAIT_FULL);
                *reinterpret_cast<volatile int*>(&s_abort) = 1;
            }
            tc_commit(o_done);
        }
    } else if (warp >= 8) {
        // ---- converters
        const int ctid = tid - 256;
        bool ok = true;
        for (int c = 0; c < 2 * n && ok; c++) {
            const int side = c & 1, slot = c % 3;
            ok = mbar_wait_bounded(p.ctl.wait_cycles, &raw_full[slot], (c / 3) & 1);
            if (ok && c >= 3) ok = mbar_wait_bounded(p.ctl.wait_cycles, &kv_free[slot], ((c / 3) - 1) & 1);
            if (!ok) break;
            if (QK8 && side == 0) {
                // the K side goes to the tensor cores as it is: the codes, already K-major under the 128-byte swizzle, are
                // copied into the operand buffer (so that buffers and barriers turn over as in the other variant), and the
                // keys' factors kscale / sqrt(D) are set out for the ReLU² warps
                const uint4* src = reinterpret_cast<const uint4*>(raw + slot * CODE_BYTES);
                uint4* dst = reinterpret_cast<uint4*>(kvb + slot * PF_TILE16);
#pragma unroll
                for (int it = 0; it < CODE_BYTES / 16 / (PF_CONV_WARPS * 32); it++) dst[it * (PF_CONV_WARPS * 32) + ctid] = src[it * (PF_CONV_WARPS * 32) + ctid];
                const uint8_t* ksc = scl + ((c >> 1) & 1) * 1024;
                if (ctid < BLK)
                    kfac[((c >> 1) & 1) * BLK + ctid] =
                        (SB == 4 ? reinterpret_cast<const float*>(ksc)[ctid] : __half2float(reinterpret_cast<const __half*>(ksc)[ctid])) *
                        (rsqrtf(float(HD)) * PF_QK8_C0);
            } else {
                convert_side<SB>(raw + slot * CODE_BYTES, kvb + slot * PF_TILE16, ctid, scl + ((c >> 1) & 1) * 1024 + side * BLK * SB,
                                 side == 0 ? rsqrtf(float(HD)) : 1.0f);
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                if (QK8 && side == 0) mbar_arrive(&kf_ready[(c >> 1) & 1]);
                mbar_arrive(&kv_ready[slot]);
                mbar_arrive(&raw_empty[slot]);
            }
        }
        if (!ok) {
            atomicExch(p.ctl.err, ERR_WAIT_FULL);
            *reinterpret_cast<volatile int*>(&s_abort) = 1;
        }
    } else {
        // ---- ReLU² warps: warpgroup x (warps 4x .. 4x+3) owns tile x, one query row a thread
        const int x = warp >> 2, r = tid & 127;
        const uint32_t lane_sel = uint32_t((warp & 3) * 32) << 16;
        const uint32_t tS = tmem + 128 * x, tO = tmem + 256 + 128 * x;
        const int pos_r = p0 + t0[x] + r;               // this row's absolute position
        const int nx = max(0, min(je, npg[x]) - jb);     // pages of this CTA's range that the tile sees
        float rowsum = 0.0f;
        bool ok = true;
        for (int i = 0; i < nx; i++) {
            const int j = jb + i;
            ok = __all_sync(0xffffffffu, mbar_wait_bounded(p.ctl.wait_cycles, &s_full[x], i & 1) &&
                                             (!QK8 || mbar_wait_bounded(p.ctl.wait_cycles, &kf_ready[i & 1], (i >> 1) & 1)));
            if (!ok) break;   // (warp-uniform: the TMEM loads below are warp-collective)
            tc_fence_after();
            const bool diag = j * BLK + BLK - 1 > p0 + t0[x];   // some (row, key) of this page is masked
            // chunk cc + 1 of the row is on its way from TMEM while chunk cc is squared and packed
            uint32_t sbuf[2][32];
            tmem_ld32(tS + lane_sel, sbuf[0]);
            const float4* kf4 = reinterpret_cast<const float4*>(kfac + (i & 1) * BLK);
#pragma unroll
            for (int cc = 0; cc < 4; cc++) {
                uint32_t(&s)[32] = sbuf[cc & 1];
                if (cc < 3) tmem_ld32_async(tS + 32 * (cc + 1) + lane_sel, sbuf[(cc + 1) & 1]);
                if (QK8) {
                    // int32 dots -> u = S x the key's factor (one broadcast load a 4 keys). |S| < 2^22, so S + 1.5 x 2^23 as
                    // float bits is that float exactly: an integer add and a float subtract instead of a conversion (which
                    // runs at a quarter of their rate).
#pragma unroll
                    for (int e4 = 0; e4 < 8; e4++) {
                        const float4 kf = kf4[8 * cc + e4];
                        s[4 * e4 + 0] = __float_as_uint((__uint_as_float(s[4 * e4 + 0] + 0x4B400000u) - 12582912.0f) * kf.x);
                        s[4 * e4 + 1] = __float_as_uint((__uint_as_float(s[4 * e4 + 1] + 0x4B400000u) - 12582912.0f) * kf.y);
                        s[4 * e4 + 2] = __float_as_uint((__uint_as_float(s[4 * e4 + 2] + 0x4B400000u) - 12582912.0f) * kf.z);
                        s[4 * e4 + 3] = __float_as_uint((__uint_as_float(s[4 * e4 + 3] + 0x4B400000u) - 12582912.0f) * kf.w);
                    }
                }
                uint32_t pk[16];
                if (diag) {
#pragma unroll
                    for (int e = 0; e < 32; e += 2) {
                        const float m0 = fmaxf(__uint_as_float(s[e]), 0.0f), m1 = fmaxf(__uint_as_float(s[e + 1]), 0.0f);
                        float w0 = m0 * m0, w1 = m1 * m1;
                        const int kb = j * BLK + 32 * cc + e;
                        if (kb > pos_r) w0 = 0.0f;
                        if (kb + 1 > pos_r) w1 = 0.0f;
                        rowsum += w0 + w1;
                        pk[e >> 1] = pack_h2(w0, w1);
                    }
                } else {
                    // unmasked pages (all but the last one or two of a tile): ReLU² on packed fp16 pairs. The 16
                    // products a half accumulates stay far inside fp16; their sum joins the fp32 row sum once a chunk.
                    const __half2 zero = __float2half2_rn(0.0f);
                    __half2 part = zero;
#pragma unroll
                    for (int e = 0; e < 32; e += 2) {
                        __half2 hm = __hmax2(__floats2half2_rn(__uint_as_float(s[e]), __uint_as_float(s[e + 1])), zero);
                        hm = __hmul2(hm, hm);
                        part = __hadd2(part, hm);
                        pk[e >> 1] = *reinterpret_cast<uint32_t*>(&hm);
                    }
                    const float2 pf = __half22float2(part);
                    rowsum += pf.x + pf.y;
                }
                // P (fp16) goes over the S columns already consumed: chunk cc's 16 columns lie inside [0, 32 cc + 32)
                tmem_st16(tS + 16 * cc + lane_sel, pk);
                if (cc < 3) tmem_ld_arrived(sbuf[(cc + 1) & 1]);
            }
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_ready[x]);
        }
        if (ok) ok = mbar_wait_bounded(p.ctl.wait_cycles, o_done, 0);
        ok = __all_sync(0xffffffffu, ok);   // (warp-uniform: the TMEM loads below are warp-collective)
        if (!ok) {
            atomicExch(p.ctl.err, ERR_WAIT_FULL);
            *reinterpret_cast<volatile int*>(&s_abort) = 1;
        }
        if (nparts > 1 && !p.cls) {
            // The page ranges of the unit meet in the scratch (common.metal:88-99). Each range's CTA announces itself on the
            // unit's first counter when its products are complete; all but the last to do so leave their unnormalised O and
            // row sums in their slot and say so on the second counter. The last waits (bounded) for those, adds the ranges in
            // range order, its own straight from TMEM, and writes the rows: it writes no partial and nothing is staged in
            // shared memory. All eight warps pass both barriers below, also one whose wait ran out.
            // With many ranges a unit (p.reduce_later) none of this happens: every range leaves its partial, the first one with
            // the sink of the denominator in its row sums, and prefill_reduce_kernel, next in the stream, adds them.
            tc_fence_after();
            int* arrived = p.counters + unit;
            int* written = p.counters + p.units + unit;
            if (tid == 0 && !p.reduce_later) s_last = atomicAdd(arrived, 1) == nparts - 1;
            if (!p.reduce_later) relu_warps_sync();
            const bool last = !p.reduce_later && s_last != 0;
            const size_t tstride = size_t(BLK) * (HD + 1);   // floats of a tile's partial: column-major [128 + 1][128 rows]
            if (p.reduce_later) {
                float* pcol = p.partials + (size_t(slot0 + split) * 2 + x) * tstride + r;
                if (ok) {
#pragma unroll 1
                    for (int cc = 0; cc < 4; cc++) {
                        uint32_t acc[32];
                        if (nx > 0) tmem_ld32(tO + 32 * cc + lane_sel, acc);
#pragma unroll
                        for (int e = 0; e < 32; e++) pcol[size_t(32 * cc + e) * BLK] = nx > 0 ? __uint_as_float(acc[e]) : 0.0f;
                    }
                    pcol[size_t(HD) * BLK] = split == 0 ? sqrtf(float(HD)) * PF_PSCALE * (QK8 ? qsc[x * BLK + r] : 1.0f) + rowsum : rowsum;
                }
            } else if (!last) {
                // the 32 rows of a warp write 32 consecutive floats of a column
                float* pcol = p.partials + (size_t(slot0 + split) * 2 + x) * tstride + r;
                if (ok) {
#pragma unroll 1
                    for (int cc = 0; cc < 4; cc++) {
                        uint32_t acc[32];
                        if (nx > 0) tmem_ld32(tO + 32 * cc + lane_sel, acc);
#pragma unroll
                        for (int e = 0; e < 32; e++) pcol[size_t(32 * cc + e) * BLK] = nx > 0 ? __uint_as_float(acc[e]) : 0.0f;
                    }
                    pcol[size_t(HD) * BLK] = rowsum;
                }
                __threadfence();
                relu_warps_sync();
                if (tid == 0 && p.ctl.stall_at != EMBLA_STALL_PARTIALS) atomicAdd(written, 1);   // (unless the diagnostic stall withholds it)
            } else {
                if (tid == 0) {
                    bool seen = false;
                    const long long c0 = clock64();
                    for (uint32_t i = 0; i < WAIT_LIMIT && !seen; i++) {
                        seen = ld_acquire_gpu(written) >= nparts - 1;
                        if (!seen && clock64() - c0 > p.ctl.wait_cycles) break;
                    }
                    if (!seen) {
                        atomicExch(p.ctl.err, ERR_WAIT_FULL);
                        *reinterpret_cast<volatile int*>(&s_abort) = 1;
                    }
                    *arrived = 0;    // (every range of the unit has been at both counters: they are left at zero for the next launch)
                    *written = 0;
                }
                relu_warps_sync();
                if (ok && !*reinterpret_cast<volatile int*>(&s_abort)) {
                    const float* pbase = p.partials + (size_t(slot0) * 2 + x) * tstride + r;   // range 0; range s is 2 tstride x s on
                    float den = sqrtf(float(HD)) * PF_PSCALE * (QK8 ? qsc[x * BLK + r] : 1.0f);
                    for (int sp = 0; sp < nparts; sp++) den += sp == split ? rowsum : __ldcg(pbase + size_t(sp) * 2 * tstride + size_t(HD) * BLK);
                    const float inv = 1.0f / den;
                    const size_t ooff = size_t(b) * p.o_seq_stride + size_t(t0[x] + r) * p.o_token_stride + size_t(h) * HD;
                    uint16_t* orow = static_cast<uint16_t*>(p.o) + ooff;
#pragma unroll 1
                    for (int cc = 0; cc < 4; cc++) {
                        float tot[32];
#pragma unroll
                        for (int e = 0; e < 32; e++) tot[e] = 0.0f;
#pragma unroll 1
                        for (int sp = 0; sp < nparts; sp++) {
                            uint32_t v[32];
                            if (sp == split) {
                                if (nx > 0) tmem_ld32(tO + 32 * cc + lane_sel, v);
                                else {
#pragma unroll
                                    for (int e = 0; e < 32; e++) v[e] = 0u;
                                }
                            } else {
                                const float* pc = pbase + size_t(sp) * 2 * tstride + size_t(32 * cc) * BLK;
#pragma unroll
                                for (int e = 0; e < 32; e++) v[e] = __float_as_uint(__ldcg(pc + size_t(e) * BLK));
                            }
#pragma unroll
                            for (int e = 0; e < 32; e++) tot[e] += __uint_as_float(v[e]);
                        }
                        if (r < rows[x]) {
                            uint32_t outw[16];
#pragma unroll
                            for (int e = 0; e < 32; e += 2) {
                                if (DT == EMBLA_F16) outw[e >> 1] = pack_h2(tot[e] * inv, tot[e + 1] * inv);
                                else {
                                    __nv_bfloat162 t = __floats2bfloat162_rn(tot[e] * inv, tot[e + 1] * inv);
                                    outw[e >> 1] = *reinterpret_cast<uint32_t*>(&t);
                                }
                            }
#pragma unroll
                            for (int v4 = 0; v4 < 4; v4++) {
                                const uint4 val = make_uint4(outw[4 * v4], outw[4 * v4 + 1], outw[4 * v4 + 2], outw[4 * v4 + 3]);
                                *reinterpret_cast<uint4*>(orow + 32 * cc + 8 * v4) = val;
                                for (int pr = 0; pr < p.n_peers; pr++)
                                    *reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.o_peer[pr]) + ooff + 32 * cc + 8 * v4) = val;
                            }
                        }
                    }
                }
            }
        } else if (!ok) {
        } else if (nparts > 1) {
            // cluster: this CTA's partial stays in its own shared memory (everything from the query tiles on is free once the
            // last product has completed), row-major [2 tiles][128 rows][128 + 1], for the cluster to read
            tc_fence_after();
            float* prow = reinterpret_cast<float*>(smem) + size_t(x * BLK + r) * (HD + 1);
#pragma unroll 1
            for (int cc = 0; cc < 4; cc++) {
                uint32_t acc[32];
                if (nx > 0) tmem_ld32(tO + 32 * cc + lane_sel, acc);
#pragma unroll
                for (int e = 0; e < 32; e++) prow[32 * cc + e] = nx > 0 ? __uint_as_float(acc[e]) : 0.0f;
            }
            prow[HD] = rowsum;
        } else if (nx > 0) {
            tc_fence_after();
            const float inv = 1.0f / (sqrtf(float(HD)) * PF_PSCALE * (QK8 ? qsc[x * BLK + r] : 1.0f) + rowsum);
            const size_t ooff = size_t(b) * p.o_seq_stride + size_t(t0[x] + r) * p.o_token_stride + size_t(h) * HD;
            uint16_t* orow = static_cast<uint16_t*>(p.o) + ooff;
#pragma unroll 1
            for (int cc = 0; cc < 4; cc++) {
                uint32_t acc[32];
                tmem_ld32(tO + 32 * cc + lane_sel, acc);
                if (r < rows[x]) {
                    uint32_t outw[16];
#pragma unroll
                    for (int e = 0; e < 32; e += 2) {
                        const float a0 = __uint_as_float(acc[e]) * inv, a1 = __uint_as_float(acc[e + 1]) * inv;
                        if (DT == EMBLA_F16) outw[e >> 1] = pack_h2(a0, a1);
                        else {
                            __nv_bfloat162 t = __floats2bfloat162_rn(a0, a1);
                            outw[e >> 1] = *reinterpret_cast<uint32_t*>(&t);
                        }
                    }
#pragma unroll
                    for (int v4 = 0; v4 < 4; v4++)
                    {
                        const uint4 val = make_uint4(outw[4 * v4], outw[4 * v4 + 1], outw[4 * v4 + 2], outw[4 * v4 + 3]);
                        *reinterpret_cast<uint4*>(orow + 32 * cc + 8 * v4) = val;
                        for (int pr = 0; pr < p.n_peers; pr++)   // the same 16 bytes into every peer's copy (NVLink stores)
                            *reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.o_peer[pr]) + ooff + 32 * cc + 8 * v4) = val;
                    }
                }
            }
        }
    }
    if (nparts > 1 && p.cls) {
        // Cluster combine: after one cluster barrier every range's partial is complete in its CTA's shared memory; the CTA of
        // rank k then owns a slice of the rows of both tiles and adds the cluster's ranges in order over distributed shared
        // memory (common.metal:88-99, without a last arriver: every SM of the cluster takes a share). A second barrier
        // keeps every CTA's shared memory alive until its peers have read it.
        const int cl = p.cls, rank = split;
        cluster_arrive();
        cluster_wait();
        const int R = (BLK + cl - 1) / cl;                           // rows of a tile this CTA finishes
        float* den = reinterpret_cast<float*>(smem + (2 + PF_KVBUFS) * PF_TILE16);   // [2][R], behind the partial
        const uint32_t part0 = smem_u32(smem);
        {
            // (the loads of an element from all ranges are issued before the first is used: each crosses the SM-to-SM network)
            for (int i = tid; i < 2 * R; i += PF_THREADS) {
                const int x = i / R, r = rank * R + i % R;
                if (r >= BLK) continue;
                float v[8];
#pragma unroll
                for (int sp = 0; sp < 8; sp++)
                    v[sp] = sp < cl ? cluster_ld_f32(cluster_map(part0 + uint32_t((x * BLK + r) * (HD + 1) + HD) * 4u, uint32_t(sp))) : 0.0f;
                float sum = 0.0f;
#pragma unroll
                for (int sp = 0; sp < 8; sp++) sum += v[sp];
                den[i] = sqrtf(float(HD)) * PF_PSCALE * (QK8 ? qsc[x * BLK + r] : 1.0f) + sum;
            }
            __syncthreads();
            for (int it = tid; it < 2 * R * (HD / 2); it += PF_THREADS) {
                const int i = it / (HD / 2), c = 2 * (it % (HD / 2));
                const int x = i / R, r = rank * R + i % R;
                if (r >= rows[x]) continue;
                const uint32_t at = part0 + uint32_t((x * BLK + r) * (HD + 1) + c) * 4u;
                float v0[8], v1[8];
#pragma unroll
                for (int sp = 0; sp < 8; sp++) {
                    const uint32_t ra = cluster_map(at, uint32_t(sp < cl ? sp : 0));
                    v0[sp] = sp < cl ? cluster_ld_f32(ra) : 0.0f;
                    v1[sp] = sp < cl ? cluster_ld_f32(ra + 4u) : 0.0f;
                }
                float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
                for (int sp = 0; sp < 8; sp++) {
                    a0 += v0[sp];
                    a1 += v1[sp];
                }
                const float inv = 1.0f / den[i];
                uint32_t w;
                if (DT == EMBLA_F16) w = pack_h2(a0 * inv, a1 * inv);
                else {
                    __nv_bfloat162 t = __floats2bfloat162_rn(a0 * inv, a1 * inv);
                    w = *reinterpret_cast<uint32_t*>(&t);
                }
                const size_t off = size_t(b) * p.o_seq_stride + size_t(t0[x] + r) * p.o_token_stride + size_t(h) * HD + c;
                *reinterpret_cast<uint32_t*>(static_cast<uint16_t*>(p.o) + off) = w;
                for (int pr = 0; pr < p.n_peers; pr++) *reinterpret_cast<uint32_t*>(static_cast<uint16_t*>(p.o_peer[pr]) + off) = w;
            }
            cluster_arrive();
            cluster_wait();
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == PF_MMA) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

// Balanced launch (fewer units than SMs, too many for a split into equal ranges to fill the SMs). The pages of all units,
// laid end to end in unit order, are cut into `runs` equal runs (one an SM) and again wherever a unit ends: every piece (one
// or two a run) is the work of one CTA, and a unit's pieces meet in the scratch like the ranges of a split. The CTAs take
// the pieces longest first: as the SMs that drew the shortest of the long pieces come free, they get the longest of the short
// ones, and every SM ends up with about a run's worth of pages. This kernel (ahead of the attention kernel in the stream,
// which may become resident meanwhile and waits for it) lays the pieces out from the chunk positions: pieces[k] is the work
// of CTA k. Each of its CTAs works the whole layout out and places 32 of the pieces, sixteen threads counting the longer
// pieces of each.
struct PfPiece {
    int unit, split, nparts, slot0, jb, je, n_pieces, pad;
};

__global__ void __launch_bounds__(512) prefill_pieces_kernel(const int32_t* pos0, int n_tokens, int pairs, int heads, int units, int runs,
                                                             PfPiece* pieces, int2* unit_slots) {
    __shared__ int pre[PF_BAL_UNITS + 1], slot[PF_BAL_UNITS + 1], size[PF_BAL_PIECES];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int U = units, G = runs;
    pdl_launch_dependents();
    auto scan256 = [&](int* a, int nn) {   // (warp 0) inclusive prefix sums of a[0 .. nn), nn <= 256
        int v[8], sum = 0;
#pragma unroll
        for (int k = 0; k < 8; k++) {
            v[k] = lane * 8 + k < nn ? a[lane * 8 + k] : 0;
            sum += v[k];
        }
        int incl = sum;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += t;
        }
        int run = incl - sum;
#pragma unroll
        for (int k = 0; k < 8; k++) {
            run += v[k];
            if (lane * 8 + k < nn) a[lane * 8 + k] = run;
        }
    };
    // pages the later tile of unit u sees
    for (int u = tid; u < U; u += blockDim.x) {
        const int px = u % pairs, bb = u / (pairs * heads);
        pre[u + 1] = (pos0[bb] + min(n_tokens, (2 * px + 2) * BLK) - 1) / BLK + 1;
    }
    if (tid == 0) pre[0] = slot[0] = 0;
    __syncthreads();
    if (warp == 0) scan256(pre + 1, U);
    __syncthreads();
    const unsigned T = unsigned(pre[U]);
    // run c holds pages [c T / G, (c + 1) T / G) (the host keeps T x G inside 32 bits); the last run that starts at or
    // before page x:
    auto run_of = [&](int x) { return int((unsigned(x + 1) * unsigned(G) + T - 1) / T) - 1; };
    auto run_start = [&](int c) { return int(unsigned(c) * T / unsigned(G)); };
    for (int u = tid; u < U; u += blockDim.x) slot[u + 1] = run_of(pre[u + 1] - 1) - run_of(pre[u]) + 1;
    __syncthreads();
    if (warp == 0) scan256(slot + 1, U);
    __syncthreads();
    const int S = slot[U];   // pieces in all: at most U + G - 1
    if (blockIdx.x == 0 && unit_slots)
        for (int u = tid; u < U; u += blockDim.x) unit_slots[u] = make_int2(slot[u], slot[u + 1] - slot[u]);
    // piece t is part t - slot[u] of the unit u it falls in (the last u with slot[u] <= t)
    auto piece = [&](int t) {
        int lo = 0, hi = U - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (slot[mid] <= t) lo = mid;
            else hi = mid - 1;
        }
        const int u = lo, part = t - slot[u], c = run_of(pre[u]) + part;
        PfPiece pc;
        pc.unit = u;
        pc.split = part;
        pc.nparts = slot[u + 1] - slot[u];
        pc.slot0 = slot[u];
        pc.jb = max(run_start(c), pre[u]) - pre[u];
        pc.je = min(run_start(c + 1), pre[u + 1]) - pre[u];
        pc.n_pieces = S;
        pc.pad = 0;
        return pc;
    };
    for (int t = tid; t < S; t += blockDim.x) {
        const PfPiece pc = piece(t);
        size[t] = pc.je - pc.jb;
    }
    __syncthreads();
    // this CTA's 32 pieces: piece t goes to the place that counts the pieces ahead of it (longer, or as long and earlier)
    const int t = int(blockIdx.x) * 32 + (tid >> 4), sub = tid & 15;
    const int sz = t < S ? size[t] : 0;
    int rank = 0;
    for (int j = sub; j < S; j += 16) {
        const int other = size[j];
        rank += (other > sz) || (other == sz && j < t);
    }
#pragma unroll
    for (int d = 8; d >= 1; d >>= 1) rank += __shfl_xor_sync(0xffffffffu, rank, d, 16);
    if (sub == 0 && t < S) pieces[rank] = piece(t);
    if (sub == 0 && t >= S && t < U + G - 1) {
        // (CTAs of the attention kernel past the last piece find this and leave)
        PfPiece none = {};
        none.n_pieces = S;
        pieces[t] = none;
    }
}

// Adds the partial sums that the ranges of every unit left in the scratch (p.reduce_later) and writes the rows: a CTA takes 32
// rows of one tile of one unit. Its warps read the ranges' columns with the lanes across the rows (coalesced: a partial is
// column-major), add them in range order into a padded tile in shared memory, and write each row with the lanes across the
// head dims (common.metal:88-99, shared out over many SMs instead of a unit's last CTA).
template <int DT>
__global__ void __launch_bounds__(256) prefill_reduce_kernel(const __grid_constant__ PrefillParams p) {
    __shared__ __align__(16) float tile[32][HD + 4];   // column HD: the denominator (rows 16-byte aligned)
    pdl_wait();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rb = blockIdx.x, x = blockIdx.y, unit = blockIdx.z;
    const int pair_ix = unit % p.pairs, h = (unit / p.pairs) % p.heads, b = unit / (p.pairs * p.heads);
    const int t0 = (2 * pair_ix + x) * BLK, rows = max(0, min(BLK, p.n_tokens - t0));
    if (32 * rb >= rows) return;
    int slot0 = unit * p.nsplit, nparts = p.nsplit;
    if (p.balanced) {
        const int2 us = p.unit_slots[unit];
        slot0 = us.x;
        nparts = us.y;
    }
    if (nparts <= 1) return;   // (a unit inside one run of a balanced launch: its CTA has written the rows itself)
    const size_t tstride = size_t(BLK) * (HD + 1);
    const float* base = p.partials + (size_t(slot0) * 2 + x) * tstride + 32 * rb + lane;
    // a warp takes columns warp, warp + 8, ...: four columns at a time, the ranges' loads of each in flight together
    for (int c0 = warp; c0 <= HD; c0 += 32) {
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int sp0 = 0; sp0 < nparts; sp0 += 4) {
            float v[4][4];
#pragma unroll
            for (int k = 0; k < 4; k++)
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int c = c0 + 8 * k;
                    v[k][u] = (c <= HD && sp0 + u < nparts) ? __ldcg(base + size_t(sp0 + u) * 2 * tstride + size_t(c) * BLK) : 0.0f;
                }
#pragma unroll
            for (int k = 0; k < 4; k++)
#pragma unroll
                for (int u = 0; u < 4; u++) acc[k] += v[k][u];
        }
#pragma unroll
        for (int k = 0; k < 4; k++)
            if (c0 + 8 * k <= HD) tile[lane][c0 + 8 * k] = acc[k];
    }
    __syncthreads();
    for (int rr = warp; rr < 32; rr += 8) {
        const int r = 32 * rb + rr;
        if (r >= rows) break;
        const float inv = 1.0f / tile[rr][HD];
        const size_t off = size_t(b) * p.o_seq_stride + size_t(t0 + r) * p.o_token_stride + size_t(h) * HD + 4 * lane;
        const float4 v = *reinterpret_cast<const float4*>(&tile[rr][4 * lane]);
        uint2 w;
        if (DT == EMBLA_F16) {
            w.x = pack_h2(v.x * inv, v.y * inv);
            w.y = pack_h2(v.z * inv, v.w * inv);
        } else {
            __nv_bfloat162 t0b = __floats2bfloat162_rn(v.x * inv, v.y * inv), t1b = __floats2bfloat162_rn(v.z * inv, v.w * inv);
            w.x = *reinterpret_cast<uint32_t*>(&t0b);
            w.y = *reinterpret_cast<uint32_t*>(&t1b);
        }
        *reinterpret_cast<uint2*>(static_cast<uint16_t*>(p.o) + off) = w;
        for (int pr = 0; pr < p.n_peers; pr++) *reinterpret_cast<uint2*>(static_cast<uint16_t*>(p.o_peer[pr]) + off) = w;
    }
}

template <int DT, int SB, bool QK8>
__global__ void __launch_bounds__(PF_THREADS, 1) full_prefill_kernel(const __grid_constant__ CUtensorMap tmap,
                                                                     const __grid_constant__ PrefillParams p) {
    PfSegment sg;
    if (p.balanced) {
        pdl_wait();   // for the kernel that lays the pieces out
        const int4* e = reinterpret_cast<const int4*>(p.pieces + blockIdx.x);
        const int4 a = __ldcg(e), c = __ldcg(e + 1);   // unit, split, nparts, slot0 | jb, je, pieces in all
        if (int(blockIdx.x) >= c.z) return;
        sg.pair_ix = a.x % p.pairs;
        sg.h = (a.x / p.pairs) % p.heads;
        sg.b = a.x / (p.pairs * p.heads);
        sg.split = a.y;
        sg.nparts = a.z;
        sg.slot0 = a.w;
        sg.jb = c.x;
        sg.je = c.y;
    } else {
        // split-KV: ReLU² partial sums of page ranges just add
        sg.h = blockIdx.y;
        sg.b = blockIdx.z;
        sg.pair_ix = blockIdx.x / p.nsplit;
        sg.split = blockIdx.x % p.nsplit;
        sg.nparts = p.nsplit;
        const int unit = (sg.b * p.heads + sg.h) * p.pairs + sg.pair_ix;
        const int n_all = (p.pos0[sg.b] + min(p.n_tokens, (2 * sg.pair_ix + 2) * BLK) - 1) / BLK + 1;   // pages the later tile sees
        const int pps = (n_all + p.nsplit - 1) / p.nsplit;
        sg.jb = sg.split * pps;
        sg.je = min(n_all, sg.jb + pps);
        sg.slot0 = unit * p.nsplit;
    }
    full_prefill_segment<DT, SB, QK8>(tmap, p, sg);
}

}  // namespace embla

using namespace embla;

// bytes of one (unit, page range) slot of partial sums: two tiles of [128 + 1 columns][128 rows] fp32
static constexpr size_t PF_SLOT_BYTES = size_t(2) * BLK * (HD + 1) * sizeof(float);

extern "C" EmblaStatus embla_attn_reserve_prefill(EmblaAttn* ctx, void* stream) {
    if (!ctx) EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_reserve_prefill: null context");
    if (ctx->prefill_scratch) return EMBLA_OK;
    // A split pays only while the CTAs fit one wave or two: two slots an SM, two counters a unit (a multiple of four, so
    // that the piece table of a balanced launch behind them starts on 16 bytes).
    const size_t slots = 2 * size_t(ctx->sm_count), counters = (2 * size_t(ctx->sm_count) + 3) & ~size_t(3);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    EMBLA_CUDA_TRY(cudaMalloc(&ctx->prefill_scratch, slots * PF_SLOT_BYTES + counters * sizeof(int) + PF_BAL_PIECES * sizeof(PfPiece) + PF_BAL_UNITS * sizeof(int2)));
    EMBLA_CUDA_TRY(cudaMemsetAsync(ctx->prefill_scratch + slots * PF_SLOT_BYTES, 0, counters * sizeof(int), s));
    ctx->prefill_scratch_bytes = slots * PF_SLOT_BYTES;
    ctx->prefill_counters = int(counters);
    return EMBLA_OK;
}

template <int DT, int SB, bool QK8>
static EmblaStatus launch_prefill(EmblaAttn* ctx, const EmblaKVPool* pool, PrefillParams& p, int batch, int max_pages, cudaStream_t s) {
    auto kern = full_prefill_kernel<DT, SB, QK8>;
    static bool configured[64] = {};
    if (!configured[ctx->device & 63]) {
        EMBLA_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(PF_SMEM)));
        configured[ctx->device & 63] = true;
    }
    // A unit = 256 tokens of one head. With fewer units than SMs (short chunks, few heads on this GPU) the pages of
    // a unit are shared among several CTAs whose partial sums are added up (ReLU² partials are additive).
    const int pairs = (p.n_tokens + 2 * BLK - 1) / (2 * BLK);
    const int units = pairs * ctx->cfg.n_q_heads * batch;
    // Page ranges per unit: the even split that minimises (waves of CTAs over the SMs) x (pages of a range + the fixed cost
    // of a CTA), against the balanced launch further down. Two ways for the ranges of an even split to meet (ReLU² partials
    // are additive), costs in half pages' worth as measured on the shards of config 3 (a page is 1.8 us of a CTA):
    //   ns ranges through global scratch: 4 for a lone CTA (query load, TMEM set-up, pipeline fill); split, 10 and 4 for every
    //     other range when the unit's last range adds them, 16 and 6 for the reduce kernel when that does (below);
    //   the ranges as one thread-block cluster of cl <= 8 CTAs, added over distributed shared memory, every CTA finishing a
    //     slice of the rows: about 18 + cl / 2, and no scratch.
    // A cluster split is taken only in as many waves as cudaOccupancyMaxActiveClusters says the GPU holds at once (a
    // cluster needs its SMs inside one GPC: 15 clusters of 8 CTAs of this kernel, 213 KB of shared memory each, 33 of 4, 74
    // of 2); EMBLA_NO_CLUSTER=1 turns clusters off. Several clusters a unit, their slices meeting in the scratch, measured
    // no faster than plain ranges through the scratch (16 units: 86-93 us either way; the CTAs of a unit finish up to 16 us
    // apart, which either combine waits out) and are not kept. Ranges hold at least 8 pages; at most 16 ranges. The scratch
    // is what embla_attn_reserve_prefill allocated (this call never allocates or synchronises): a split through it is taken
    // only as far as it holds; without a reserve only lone CTAs and clusters remain.
    const long slots = long(ctx->prefill_scratch_bytes / PF_SLOT_BYTES);
    const char* ncl_env = getenv("EMBLA_NO_CLUSTER");
    const bool use_clusters = !(ncl_env && ncl_env[0] == '1');
    static int max_clusters[64][9] = {};     // per device and cluster size; 0 = not asked yet, -1 = none
    auto clusters_at_once = [&](int cl) {
        int& mc = max_clusters[ctx->device & 63][cl];
        if (mc == 0) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(cl, 1, 1);
            cfg.blockDim = dim3(PF_THREADS);
            cfg.dynamicSmemBytes = PF_SMEM;
            cudaLaunchAttribute at;
            at.id = cudaLaunchAttributeClusterDimension;
            at.val.clusterDim.x = unsigned(cl);
            at.val.clusterDim.y = 1;
            at.val.clusterDim.z = 1;
            cfg.attrs = &at;
            cfg.numAttrs = 1;
            int n = 0;
            mc = (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) == cudaSuccess && n > 0) ? n : -1;
            (void)cudaGetLastError();
        }
        return mc;
    };
    // Ranges that meet in the scratch are added by the unit's last range in its epilogue while they are few; from four ranges
    // a unit on every range only leaves its partial and prefill_reduce_kernel, launched behind, adds them on many SMs (8 half
    // pages a range for the query tiles and the partial, 6 for that kernel; one CTA adding eight others' partials alone took
    // 25 us). EMBLA_PREFILL_REDUCE=0 / 1 takes the first / second way regardless.
    const char* red_env = getenv("EMBLA_PREFILL_REDUCE");
    const int reduce_mode = red_env ? atoi(red_env) : -1;
    auto reduce_for = [&](long ranges) { return reduce_mode < 0 ? ranges >= 4 : reduce_mode == 1; };
    int nsplit = 1, cls = 0;
    bool reduce_later = false;
    long best = -1;
    for (int cl = 1; cl <= (use_clusters ? 8 : 1); cl++) {
        for (int ng = 1; cl * ng <= 16; ng++) {
            const int ns = cl * ng;
            if (ns > 1 && max_pages / ns < 8) break;
            if (cl > 1 && ng > 1) break;                                              // a cluster holds all ranges of its unit
            if (ng > 1 && (long(units) * ng > slots || 2 * units > ctx->prefill_counters)) break;   // the ranges meet in the scratch
            long waves;
            if (cl == 1) {
                waves = (long(units) * ns + ctx->sm_count - 1) / ctx->sm_count;
            } else {
                const int mc = clusters_at_once(cl);
                if (mc <= 0) break;
                waves = (long(units) * ng + mc - 1) / mc;
            }
            const bool red = cl == 1 && ns > 1 && reduce_for(ns);
            const long fixed2 = ns == 1 ? 4 : (cl == 1 ? (red ? 16 : 10 + 4 * (ns - 1)) : 18 + cl / 2);   // in half pages
            const long cost = waves * (2 * ((max_pages + ns - 1) / ns) + fixed2) + (red ? 6 : 0);
            if (best < 0 || cost < best) {
                best = cost;
                nsplit = ns;
                cls = cl > 1 ? cl : 0;
                reduce_later = red;
            }
        }
    }
    // The balanced launch (prefill_pieces_kernel): the units' pages in one run an SM, a CTA for every piece of a run that
    // lies inside one unit (at most units + SMs - 1 of them, each with a slot in the scratch), taken longest first. An SM
    // then works through a run's worth of pages in two pieces. Costs as measured on config 3 and its shards, in half pages:
    // 8 a piece (table entry, query tiles, the partial written or the rows finished, the gap between two CTAs of an SM), 2
    // for every other piece of its unit that the last piece adds, 5 for the kernel that lays the pieces out. 128 units (one
    // GPU): 0.460 ms against 0.505 with a CTA a unit on the same GPU; 64 units: 0.247 against 0.267; from 32 units down the
    // cluster split stays ahead. EMBLA_PREFILL_BALANCED=0 turns it off, =1 takes it wherever it fits.
    const char* bal_env = getenv("EMBLA_PREFILL_BALANCED");
    const int balanced_mode = bal_env ? atoi(bal_env) : -1;
    bool balanced = false;
    const int runs = ctx->sm_count;
    if (balanced_mode != 0 && units > 1 && units < runs && units <= PF_BAL_UNITS && units + runs - 1 <= PF_BAL_PIECES &&
        long(units) + runs - 1 <= slots && 2 * units <= ctx->prefill_counters && (long(units) * max_pages + 1) * runs < (1L << 31) &&
        (balanced_mode == 1 || long(units) * max_pages >= 16L * runs)) {
        const long run = (long(units) * max_pages + runs - 1) / runs;
        const long others2 = 2L * (runs - 1) / units;                 // twice the other pieces of a unit
        const bool red = reduce_for((runs - 1) / units + 2);          // (the most pieces a unit is cut into)
        const long cost = 2 * run + 2 * (8 + (red ? 0 : others2)) + 5 + (red ? 6 : 0);
        balanced = balanced_mode == 1 || cost < best;
        if (balanced) reduce_later = red;
    }
    if (balanced) {
        nsplit = 1;
        cls = 0;
    }
    p.nsplit = nsplit;
    p.cls = cls;
    p.heads = ctx->cfg.n_q_heads;
    p.pairs = pairs;
    p.units = units;
    p.balanced = balanced ? 1 : 0;
    p.reduce_later = reduce_later ? 1 : 0;
    p.unit_slots = nullptr;
    p.pieces = nullptr;
    p.partials = nullptr;
    p.counters = nullptr;
    if (balanced || (nsplit > 1 && !cls)) {
        // the counters sit after the partials and are left at zero by every launch
        p.partials = reinterpret_cast<float*>(ctx->prefill_scratch);
        p.counters = reinterpret_cast<int*>(ctx->prefill_scratch + ctx->prefill_scratch_bytes);
    }
    dim3 grid(pairs * nsplit, ctx->cfg.n_q_heads, batch);
    static const bool use_pdl = []() { const char* e = getenv("EMBLA_NO_PDL"); return !(e && e[0] == '1'); }();
    if (balanced) {
        // the piece table sits behind the counters
        PfPiece* pieces = reinterpret_cast<PfPiece*>(ctx->prefill_scratch + ctx->prefill_scratch_bytes + size_t(ctx->prefill_counters) * sizeof(int));
        p.unit_slots = reinterpret_cast<int2*>(pieces + PF_BAL_PIECES);   // (and the units' slots behind that)
        prefill_pieces_kernel<<<(units + runs - 1 + 31) / 32, 512, 0, s>>>(p.pos0, p.n_tokens, pairs, p.heads, units, runs, pieces, p.unit_slots);
        EMBLA_CUDA_TRY(cudaGetLastError());
        p.pieces = pieces;
        grid = dim3(units + runs - 1, 1, 1);
        EMBLA_CUDA_TRY(launch_kernel(use_pdl, kern, grid, dim3(PF_THREADS), PF_SMEM, s, pool->tmap_half, p));
    } else if (cls) {
        EMBLA_CUDA_TRY(launch_kernel_cluster(false, cls, kern, grid, dim3(PF_THREADS), PF_SMEM, s, pool->tmap_half, p));
    } else {
        kern<<<grid, PF_THREADS, PF_SMEM, s>>>(pool->tmap_half, p);
        EMBLA_CUDA_TRY(cudaGetLastError());
    }
    if (reduce_later)
        EMBLA_CUDA_TRY(launch_kernel(use_pdl, prefill_reduce_kernel<DT>, dim3(BLK / 32, 2, units), dim3(256), 0, s, p));
    return EMBLA_OK;
}

static EmblaStatus full_prefill_impl(EmblaAttn* ctx, const EmblaKVPool* pool, const EmblaKVView* view,
                                     const int32_t* pos0_dev, int32_t n_tokens, const EmblaQuery* q,
                                     int64_t q_token_stride, void* o_dev, int64_t o_token_stride,
                                     int64_t o_seq_stride, bool qk8, void* stream, void* const* o_peers = nullptr, int n_peers = 0) {
    if (!ctx || !pool || !view || !pos0_dev || !q || !q->q_dev || !o_dev)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_full_prefill: null argument");
    EMBLA_CHECK_DEVICE("embla_attn_full_prefill", ctx, pool);
    if (pool->kv_dtype != EMBLA_KV_INT8) EMBLA_FAIL(EMBLA_UNSUPPORTED, "embla_attn_full_prefill: the pool is not int8");
    if (pool->n_kv_heads != ctx->cfg.n_kv_heads || view->layer < 0 || view->layer >= pool->n_layers)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_full_prefill: pool/layer mismatch");
    if (view->batch <= 0 || !view->block_table_dev || n_tokens <= 0)
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_full_prefill: batch %d, n_tokens %d", view->batch, n_tokens);
    if (!q->prenormed && (q->ng != 2 || !q->g1_dev || !q->g2_dev))
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_full_prefill: the fused head norm takes both gain vectors (ng = 2)");
    if ((q_token_stride % 8) || (q->q_stride % 8) || (o_token_stride % 8) || (o_seq_stride % 8))
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_full_prefill: strides must be multiples of 8 elements (16-byte rows)");
    PrefillParams p;
    p.pool = pool->base;
    p.block_table = view->block_table_dev;
    p.pos0 = pos0_dev;
    p.q = q->q_dev;
    p.g1 = q->g1_dev;
    p.g2 = q->g2_dev;
    p.o = o_dev;
    p.n_peers = n_peers;
    for (int i = 0; i < PF_MAX_PEERS; i++) p.o_peer[i] = i < n_peers ? o_peers[i] : nullptr;
    p.ctl = kernel_ctl(ctx);
    p.q_token_stride = q_token_stride;
    p.q_seq_stride = q->q_stride;
    p.o_token_stride = o_token_stride;
    p.o_seq_stride = o_seq_stride;
    p.page_bytes = pool->page_bytes;
    p.table_stride = view->table_stride;
    p.layer = view->layer;
    p.n_layers = pool->n_layers;
    p.n_kv_heads = pool->n_kv_heads;
    p.G = ctx->cfg.n_q_heads / ctx->cfg.n_kv_heads;
    p.scale_bytes = pool->scale_bytes;
    p.rows_per_page = pool->rows_per_page;
    p.n_tokens = n_tokens;
    p.prenormed = q->prenormed;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool bf = ctx->cfg.act_dtype == EMBLA_BF16, s4 = pool->scale_bytes == 4;
    // pages a tile may see, from the caller's bound on pos0 + n_tokens (sizes the page split only)
    const int max_pages = ((view->max_seq_len > 0 ? view->max_seq_len : ctx->cfg.max_context) + BLK - 1) / BLK;
#define EMBLA_PF(DT, SB) (qk8 ? launch_prefill<DT, SB, true>(ctx, pool, p, view->batch, max_pages, s) : launch_prefill<DT, SB, false>(ctx, pool, p, view->batch, max_pages, s))
    if (bf) return s4 ? EMBLA_PF(EMBLA_BF16, 4) : EMBLA_PF(EMBLA_BF16, 2);
    return s4 ? EMBLA_PF(EMBLA_F16, 4) : EMBLA_PF(EMBLA_F16, 2);
#undef EMBLA_PF
}

extern "C" EmblaStatus embla_attn_full_prefill(EmblaAttn* ctx, const EmblaKVPool* pool, const EmblaKVView* view,
                                               const int32_t* pos0_dev, int32_t n_tokens, const EmblaQuery* q,
                                               int64_t q_token_stride, void* o_dev, int64_t o_token_stride,
                                               int64_t o_seq_stride, void* stream) {
    return full_prefill_impl(ctx, pool, view, pos0_dev, n_tokens, q, q_token_stride, o_dev, o_token_stride, o_seq_stride, false, stream);
}

extern "C" EmblaStatus embla_attn_full_prefill_scatter(EmblaAttn* ctx, const EmblaKVPool* pool, const EmblaKVView* view,
                                                       const int32_t* pos0_dev, int32_t n_tokens, const EmblaQuery* q,
                                                       int64_t q_token_stride, void* o_dev, void* const* o_peers_dev, int32_t n_peers,
                                                       int64_t o_token_stride, int64_t o_seq_stride, void* stream) {
    if (n_peers < 0 || n_peers > PF_MAX_PEERS || (n_peers > 0 && !o_peers_dev))
        EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_full_prefill_scatter: %d peers (0..%d)", n_peers, PF_MAX_PEERS);
    for (int i = 0; i < n_peers; i++)
        if (!o_peers_dev[i] || reinterpret_cast<uintptr_t>(o_peers_dev[i]) % 16)
            EMBLA_FAIL(EMBLA_BAD_ARG, "embla_attn_full_prefill_scatter: peer %d's address is null or not 16-byte aligned", i);
    return full_prefill_impl(ctx, pool, view, pos0_dev, n_tokens, q, q_token_stride, o_dev, o_token_stride, o_seq_stride, false, stream,
                             o_peers_dev, n_peers);
}

extern "C" EmblaStatus embla_attn_full_prefill_qk8(EmblaAttn* ctx, const EmblaKVPool* pool, const EmblaKVView* view,
                                                   const int32_t* pos0_dev, int32_t n_tokens, const EmblaQuery* q,
                                                   int64_t q_token_stride, void* o_dev, int64_t o_token_stride,
                                                   int64_t o_seq_stride, void* stream) {
    return full_prefill_impl(ctx, pool, view, pos0_dev, n_tokens, q, q_token_stride, o_dev, o_token_stride, o_seq_stride, true, stream);
}
