// The softmax decode kernel over 16-bit keys and values (sparse layers' gathered rows, sliding layers' rings).
// A CTA walks a contiguous range of 64-row tiles of one (sequence, kv head) through a 3-stage ring in shared
// memory, so rows are in flight while the previous tile is computed; its 4 consumer warps take 16 rows of every
// tile each. Two ways to fill a stage:
//  * gathered rows (sparse layers; rings whose size is no multiple of 64): 16-byte cp.async by the consumer
//    threads, row address from the index list / block table / ring slot;
//  * ring tiles (sliding layers): the window is cut at 64-slot boundaries of the ring, so a tile is 64 consecutive
//    ring rows and one producer thread fetches it with four TMA boxes (K and V, two 128-byte halves, 128-byte
//    swizzle), completion on the stage's mbarrier, the stage handed back through a second one; the rows of the
//    edge tiles that lie outside the window are masked. Every wait is bounded.
// S^T = K Q^T and O^T = V^T P^T are m16n8k16 tensor tiles on the data as stored; the softmax is online per warp
// (running max and sum per query head, O rescaled when the max grows), the warps merge at the end, and when a pair
// is cut into several row ranges their (max, sum, acc) partials are merged by the last CTA to arrive, in range order.
#pragma once

#include "attn16_common.cuh"

namespace embla {

constexpr int A16_THREADS = 128;                       // consumer threads; ring tiles add a producer warp
constexpr int A16_ROWS = 64;                          // rows of a tile
constexpr int A16_STAGES = 3;
constexpr int A16_SIDE = A16_ROWS * HD * 2;           // bytes of one side (K or V) of a tile: 16 KiB
constexpr int A16_STAGE = 2 * A16_SIDE;
constexpr int A16_PART = HD + 4;                      // floats per (range, head): 128 sums, max, sum
// Clusters: a head's partials are sent to the CTA that finishes it (head h: CTA h % ranges), into an inbox of
// [sender][head of this owner] rows behind the stages and queries; ranges x ceil(heads / ranges) <= 15 rows.
constexpr int A16_INBOX_ROWS = 15;
constexpr int A16_INBOX_BYTES = A16_INBOX_ROWS * A16_PART * 4;
enum { A16_SPARSE = 0, A16_SLIDING = 1, A16_FULL = 2 };
// A16_FULL: the full layers' ReLU² attention over a 16-bit cache (attn_full, attention.metal:148-220): every key of the
// sequence, weight max(s / sqrt(D), 0)², o = sum w v / (sqrt(D) + sum w). It runs through the softmax machinery with the
// running maximum pinned at zero (every rescale factor is exp(0) = 1, merges add) and the sink added where the softmax
// kernels divide. fp16 P carries the weights times 2^-6, so that a weight up to 4e6 (|s| up to 2000) still fits.
template <int DT, int MODE>
__device__ __forceinline__ float a16_pscale() { return (MODE == A16_FULL && DT == EMBLA_F16) ? 0.015625f : 1.0f; }
template <int DT, int MODE>
__device__ __forceinline__ float a16_finish(float num, float L) {
    if (MODE == A16_FULL) return num * (1.0f / a16_pscale<DT, MODE>()) / (sqrtf(float(HD)) + L);
    return num / L;
}

__device__ __forceinline__ void cons_sync() { asm volatile("bar.sync 1, %0;" ::"n"(A16_THREADS) : "memory"); }

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
    KernelCtl ctl;
    int64_t q_stride, o_stride, ring_stride;   // elements; ring_stride between sequences
    size_t page_bytes;
    int table_stride, layer, n_layers, n_kv_heads, G, prenormed, ng, ring, window;
    int max_chunks, tiles_per_cta;             // row ranges a pair is cut into, tiles in a range
    // sliding layers, fused ring write of the current token (attention.metal:47-62): its raw k, v rows or NULL
    const void* k_new;
    const void* v_new;
    const void* kgain;
    int64_t kv_stride;
    int k_prenormed;
    float rope_freq[32];
};

// CL: the ranges of a pair are the CTAs of one thread-block cluster (at most 8), launched as such; they merge their
// partials through the cluster's shared memory, each CTA finishing a share of the heads, instead of through global
// scratch and a last arriver.
template <int DT, int MODE, bool TMA, bool CL>
__global__ void __launch_bounds__(A16_THREADS + (TMA ? 32 : 0))
    attn16_decode_kernel(const Attn16Params p, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint16_t(*qs)[HD] = reinterpret_cast<uint16_t(*)[HD]>(smem + A16_STAGES * A16_STAGE);   // [8][128] activation dtype
    __shared__ uint64_t full[A16_STAGES], empty[A16_STAGES];
    __shared__ int s_last, s_failed, s_issued;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int chunk = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    trace_first(p.ctl.trace, 0);
    // Ring tiles of an "early" launch (the kernel ahead of it in the stream does not write this ring) are requested before
    // the wait for that kernel; seq_lens is an input of the whole step.
    const bool early = TMA && p.ctl.early != 0;
    const int S = p.seq_lens[b];   // (read ahead of the wait in any case: nothing on the GPU writes the sequence lengths)
    if (!early) {
        pdl_wait();
        pdl_launch_dependents();
    }
    const bool selecting = MODE == A16_SPARSE && S > EMBLA_TOPK + EMBLA_RECENT;
    const int count = MODE == A16_SLIDING ? min(S, p.window) : (selecting ? EMBLA_TOPK + EMBLA_RECENT : S);
    const int pos = S - 1;
    // Tiles: of the row list j = 0 .. count - 1 (j-th latest position for rings), or, for ring tiles, of the ring's
    // slots pos - count + 1 .. pos cut at multiples of 64 (tbase: the first such tile).
    const int tbase = TMA ? (pos - count + 1) >> 6 : 0;
    const int tiles = TMA ? (pos >> 6) - tbase + 1 : (count + A16_ROWS - 1) / A16_ROWS;
    const int nch = (tiles + p.tiles_per_cta - 1) / p.tiles_per_cta;     // ranges this sequence really has
    if (chunk >= nch) return;
    const int tile0 = chunk * p.tiles_per_cta, ntile = min(p.tiles_per_cta, tiles - tile0);

    if (TMA) {
        auto issue = [&](int t) {
            const int st = t % A16_STAGES;
            if (t == p.ctl.stall_at) return false;   // diagnostic stall: the consumers' wait for this tile runs out
            if (t >= A16_STAGES && !mbar_wait_bounded(p.ctl.wait_cycles, &empty[st], ((t / A16_STAGES) - 1) & 1)) {
                atomicExch(p.ctl.err, ERR_WAIT_EMPTY);
                return false;
            }
            uint8_t* Kt = smem + st * A16_STAGE;
            const int y = kvh * p.ring + ((tbase + tile0 + t) * A16_ROWS) % p.ring;
            mbar_expect_tx(&full[st], A16_STAGE);
            tma_load_3d(Kt, &map_k, 0, y, b, &full[st]);
            tma_load_3d(Kt + A16_ROWS * 128, &map_k, 128, y, b, &full[st]);
            tma_load_3d(Kt + A16_SIDE, &map_v, 0, y, b, &full[st]);
            tma_load_3d(Kt + A16_SIDE + A16_ROWS * 128, &map_v, 128, y, b, &full[st]);
            *reinterpret_cast<volatile int*>(&s_issued) = t + 1;
            return true;
        };
        int next = 0;
        bool issuing = true;
        if (tid == A16_THREADS) {   // the producer lane sets the barriers up itself, so that it can start before anyone else
#pragma unroll
            for (int i = 0; i < A16_STAGES; i++) {
                mbar_init(&full[i], 1);
                mbar_init(&empty[i], A16_THREADS / 32);
            }
            s_failed = 0;
            s_issued = 0;
            fence_barrier_init();
            for (; next < min(ntile, A16_STAGES) && issuing; next++) issuing = issue(next);   // the stages start empty
        }
        if (early) {
            pdl_wait();
            pdl_launch_dependents();
        }
        __syncthreads();
        if (warp == A16_THREADS / 32) {   // the producer
            if (lane == 0)
                for (; next < ntile && issuing; next++) issuing = issue(next);
            __syncwarp();
            // (a consumer that gave up a wait meets the producer here before it drains the copies in flight)
            asm volatile("bar.arrive 2, %0;" ::"n"(A16_THREADS + 32) : "memory");
            return;
        }
    }
    trace_first(p.ctl.trace, 1);

    // Gathers of tile `t` (of this CTA's range) into stage t % STAGES; every thread copies 8 chunks of K and of V. The
    // rows' addresses (index list -> block table -> page: two dependent loads) are resolved one tile ahead of their
    // use, so that those loads fly while the tile before is computed instead of stalling every warp at the issue.
    const uint8_t* const base_k = MODE == A16_SLIDING ? p.ring_k : p.pool;
    const uint8_t* const base_v = MODE == A16_SLIDING ? p.ring_v : p.pool + BLK * HD * 2;
    size_t roff[8];      // byte offsets of this thread's 8 rows of the resolved tile (this thread's 16-byte chunk included)
    uint32_t rvalid = 0;
    auto resolve_tile = [&](int t) {
        const int ch = tid & 15;
        const int jbase = (tile0 + t) * A16_ROWS;
        rvalid = 0;
#pragma unroll
        for (int it = 0; it < 8; it++) {
            const int key = it * 8 + (tid >> 4), j = jbase + key;
            const bool valid = t < ntile && j < count;
            rvalid |= uint32_t(valid) << it;
            if (MODE == A16_SLIDING) {
                const int slot = valid ? (pos - j) % p.ring : 0;
                roff[it] = (size_t(b) * p.ring_stride + (size_t(kvh) * p.ring + slot) * HD) * 2 + ch * 16;
            } else {
                int row = valid ? j : 0;
                if (selecting && valid) row = int(p.idx[(size_t(b) * p.n_kv_heads + kvh) * (EMBLA_TOPK + EMBLA_RECENT) + j]);
                const int block = p.block_table[size_t(b) * p.table_stride + (row >> 7)];
                roff[it] = ((size_t(block) * p.n_layers + p.layer) * p.n_kv_heads + kvh) * p.page_bytes + (row & 127) * (HD * 2) + ch * 16;
            }
        }
    };
    auto issue_tile = [&](int t) {   // the tile resolved last
        uint8_t* Kt = smem + (t % A16_STAGES) * A16_STAGE;
        uint8_t* Vt = Kt + A16_SIDE;
        const int ch = tid & 15, half = ch >> 3, cc = ch & 7;
#pragma unroll
        for (int it = 0; it < 8; it++) {
            const int key = it * 8 + (tid >> 4);
            const bool valid = (rvalid >> it) & 1;
            const int dst = half * (A16_ROWS * 128) + key * 128 + ((cc ^ (key & 7)) << 4);
            cp_async16(Kt + dst, base_k + roff[it], valid);
            cp_async16(Vt + dst, base_v + roff[it], valid);
        }
    };
    // Gathered rows (sparse and full layers): a row's address is two dependent loads away (index list -> block table), so the
    // three steps run a tile apart: this iteration loads the index rows of the tile five ahead, looks up the blocks of the
    // tile four ahead from the rows loaded an iteration ago, and turns the blocks loaded an iteration ago into the
    // offsets of the tile three ahead; no load is used in the iteration that issued it.
    int irow[8], bblk[8], brow[8];
    uint32_t ivalid = 0, bvalid = 0;
    auto load_rows = [&](int t) {
        ivalid = 0;
#pragma unroll
        for (int it = 0; it < 8; it++) {
            const int j = (tile0 + t) * A16_ROWS + it * 8 + (tid >> 4);
            const bool ok = t < ntile && j < count;
            ivalid |= uint32_t(ok) << it;
            irow[it] = ok ? (selecting ? int(p.idx[(size_t(b) * p.n_kv_heads + kvh) * (EMBLA_TOPK + EMBLA_RECENT) + j]) : j) : 0;
        }
    };
    auto load_blocks = [&]() {
        bvalid = ivalid;
#pragma unroll
        for (int it = 0; it < 8; it++) {
            bblk[it] = p.block_table[size_t(b) * p.table_stride + (irow[it] >> 7)];
            brow[it] = irow[it] & 127;
        }
    };
    auto make_offsets = [&]() {
        rvalid = bvalid;
#pragma unroll
        for (int it = 0; it < 8; it++)
            roff[it] = ((size_t(bblk[it]) * p.n_layers + p.layer) * p.n_kv_heads + kvh) * p.page_bytes + brow[it] * (HD * 2) + (tid & 15) * 16;
    };
    // The queries' loads go out first: their latency then overlaps the address chains below instead of following them.
    constexpr int QPW = 8 / (A16_THREADS / 32);   // heads a warp prepares
    float xq[QPW][4];
#pragma unroll
    for (int k = 0; k < QPW; k++) {
        const int hh = warp + k * (A16_THREADS / 32);
        const size_t off = size_t(b) * p.q_stride + size_t(kvh * p.G + (hh < p.G ? hh : 0)) * HD;
#pragma unroll
        for (int i = 0; i < 4; i++) xq[k][i] = hh < p.G ? Act<DT>::load(p.q, off + lane + 32 * i) : 0.0f;
    }
    if (!TMA) {
        // The first tiles' rows are resolved together: all their index loads in flight at once, then all their block-table
        // loads, then the copies (resolved tile by tile, each chain of two dependent loads would follow the one before).
        if (MODE != A16_SLIDING) {
            constexpr int PRE = A16_STAGES;   // tiles 0 .. PRE - 2 are issued here, tile PRE - 1 stays resolved for the loop,
                                              // tile PRE has its blocks on the way and tile PRE + 1 its index rows
            const int ch = tid & 15;
            int rows[PRE + 1][8];
            uint32_t valid[PRE + 1];
#pragma unroll
            for (int t = 0; t < PRE + 1; t++) {
                valid[t] = 0;
#pragma unroll
                for (int it = 0; it < 8; it++) {
                    const int j = (tile0 + t) * A16_ROWS + it * 8 + (tid >> 4);
                    const bool ok = t < ntile && j < count;
                    valid[t] |= uint32_t(ok) << it;
                    rows[t][it] = ok ? (selecting ? int(p.idx[(size_t(b) * p.n_kv_heads + kvh) * (EMBLA_TOPK + EMBLA_RECENT) + j]) : j) : 0;
                }
            }
            load_rows(PRE + 1);
            int blocks[PRE][8];
#pragma unroll
            for (int t = 0; t < PRE; t++)
#pragma unroll
                for (int it = 0; it < 8; it++) blocks[t][it] = p.block_table[size_t(b) * p.table_stride + (rows[t][it] >> 7)];
            bvalid = valid[PRE];
#pragma unroll
            for (int it = 0; it < 8; it++) {
                bblk[it] = p.block_table[size_t(b) * p.table_stride + (rows[PRE][it] >> 7)];
                brow[it] = rows[PRE][it] & 127;
            }
#pragma unroll
            for (int t = 0; t < PRE; t++) {
                rvalid = valid[t];
#pragma unroll
                for (int it = 0; it < 8; it++)
                    roff[it] = ((size_t(blocks[t][it]) * p.n_layers + p.layer) * p.n_kv_heads + kvh) * p.page_bytes +
                               (rows[t][it] & 127) * (HD * 2) + ch * 16;
                if (t < PRE - 1) {
                    if (t < ntile) issue_tile(t);
                    asm volatile("cp.async.commit_group;" ::: "memory");
                }
            }
        } else {
            resolve_tile(0);
#pragma unroll
            for (int t = 0; t < A16_STAGES - 1; t++) {
                if (t < ntile) issue_tile(t);
                asm volatile("cp.async.commit_group;" ::: "memory");
                resolve_tile(t + 1);
            }
        }
    }
    // ---- the kv head's queries (norm, RoPE for sliding layers) while the rows arrive
#pragma unroll
    for (int k = 0; k < QPW; k++) {
        const int hh = warp + k * (A16_THREADS / 32);
        if (hh < p.G && !p.prenormed) norm_rope_round<DT>(xq[k], p.g1, p.g2, p.ng, MODE == A16_SLIDING ? pos : -1, p.rope_freq, lane);
#pragma unroll
        for (int i = 0; i < 4; i++) Act<DT>::store(&qs[hh][0], lane + 32 * i, xq[k][i]);
    }
    // Sliding layers, fused ring write (attention.metal:47-62): the current token's key (normed, rotated and rounded as
    // attn_sliding does) and value come from the qkv row, not from the ring. The warp that owns the token's row of its
    // tile prepares them here, stores them to the ring slot for the steps to come and puts them into the tile below.
    // The token is row 0 of the row list, or slot pos of the last ring tile.
    const int prow = TMA ? pos & (A16_ROWS - 1) : 0;
    const int ptile = TMA ? tiles - 1 : 0;
    const bool patch = MODE == A16_SLIDING && p.k_new != nullptr && ptile >= tile0 && ptile < tile0 + ntile && warp == prow >> 4;
    float knew[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    uint16_t vnew[4] = {0, 0, 0, 0};
    if (patch) {
        const size_t off = size_t(b) * p.kv_stride + size_t(kvh) * HD;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            knew[i] = Act<DT>::load(p.k_new, off + lane + 32 * i);
            vnew[i] = reinterpret_cast<const uint16_t*>(p.v_new)[off + lane + 32 * i];
        }
        if (!p.k_prenormed) norm_rope_round<DT>(knew, p.kgain, p.kgain, 1, pos, p.rope_freq, lane);
        const size_t slot_off = size_t(b) * p.ring_stride + (size_t(kvh) * p.ring + pos % p.ring) * HD;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            Act<DT>::store(const_cast<uint8_t*>(p.ring_k), slot_off + lane + 32 * i, knew[i]);
            reinterpret_cast<uint16_t*>(const_cast<uint8_t*>(p.ring_v))[slot_off + lane + 32 * i] = vnew[i];
        }
    }
    cons_sync();

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
    trace_first(p.ctl.trace, 4);   // queries ready
    trace_last(p.ctl.trace, 6);
    const float scale = rsqrtf(float(HD));
    // running max / sum of heads 2c, 2c + 1 over this warp's rows (ReLU²: the maximum stays at zero)
    float m0 = MODE == A16_FULL ? 0.0f : NEG_BIG, m1 = m0, l0 = 0.0f, l1 = 0.0f;
    float OT[8][4];
#pragma unroll
    for (int i = 0; i < 8; i++) OT[i][0] = OT[i][1] = OT[i][2] = OT[i][3] = 0.0f;

    for (int t = 0; t < ntile; t++) {
        const int st = t % A16_STAGES;
        uint8_t* Kt = smem + st * A16_STAGE;
        uint8_t* Vt = Kt + A16_SIDE;
        if (TMA) {
            if (!__all_sync(0xffffffffu, mbar_wait_bounded(p.ctl.wait_cycles, &full[st], (t / A16_STAGES) & 1))) {
                if (lane == 0) {
                    atomicExch(p.ctl.err, ERR_WAIT_FULL);
                    *reinterpret_cast<volatile int*>(&s_failed) = 1;
                }
                break;
            }
        } else {
            asm volatile("cp.async.wait_group %0;" ::"n"(A16_STAGES - 2) : "memory");
            cons_sync();
        }
        if (t == 0) trace_last(p.ctl.trace, 7);   // the first tile has arrived
        // the 16 rows of this warp: lane holds rows r0 and r0 + 8
        const int R0 = warp * 16, r0 = R0 + rg;
        bool v0, v1;
        if (TMA) {
            const int u = (tbase + tile0 + t) * A16_ROWS + r0;   // ring position of the row
            v0 = u <= pos && u > pos - count;
            v1 = u + 8 <= pos && u + 8 > pos - count;
            // rows outside the window hold other positions or never-written memory: their weights are zero, but
            // the value rows must be finite
            const int ulo = (tbase + tile0 + t) * A16_ROWS + R0;
            if (ulo + 15 > pos || ulo <= pos - count) {
                const int zr = R0 + (lane >> 1), zu = ulo + (lane >> 1);
                if (zu > pos || zu <= pos - count) {
                    uint4* z = reinterpret_cast<uint4*>(Vt + (lane & 1) * (A16_ROWS * 128) + zr * 128);
#pragma unroll
                    for (int i = 0; i < 8; i++) z[i] = make_uint4(0, 0, 0, 0);
                }
                __syncwarp();
            }
        } else {
            const int jrow = (tile0 + t) * A16_ROWS + r0;
            v0 = jrow < count;
            v1 = jrow + 8 < count;
        }
        if (patch && tile0 + t == ptile) {
            // (only this warp reads the token's row: no other warp waits for these stores)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int d = lane + 32 * i;
                const int at = (d >> 6) * (A16_ROWS * 128) + prow * 128 + ((((d >> 3) & 7) ^ (prow & 7)) << 4) + (d & 7) * 2;
                Act<DT>::store(Kt + at, 0, knew[i]);
                *reinterpret_cast<uint16_t*>(Vt + at) = vnew[i];
            }
            __syncwarp();
        }

        // S^T = K Q^T: lane holds heads 2c and 2c + 1 of its two rows
        float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int m = 0; m < 4; m++) {
            const uint8_t* base = Kt + (m >> 1) * (A16_ROWS * 128) + r0 * 128 + (((c + 4 * (m & 1)) ^ rg) << 4);
            const uint4 x0 = *reinterpret_cast<const uint4*>(base);
            const uint4 x1 = *reinterpret_cast<const uint4*>(base + 8 * 128);
            mma16<DT>(s, x0.x, x1.x, x0.y, x1.y, qb0[2 * m], qb1[2 * m]);
            mma16<DT>(s, x0.z, x1.z, x0.w, x1.w, qb0[2 * m + 1], qb1[2 * m + 1]);
        }
        float pw[4];
        if (MODE == A16_FULL) {
            // ReLU²: no maximum, nothing to rescale; the row sums take the weights themselves, P a power of two of them
            const float a0 = fmaxf(s[0] * scale, 0.0f), a1 = fmaxf(s[1] * scale, 0.0f), a2 = fmaxf(s[2] * scale, 0.0f), a3 = fmaxf(s[3] * scale, 0.0f);
            const float w0 = v0 ? a0 * a0 : 0.0f, w1 = v0 ? a1 * a1 : 0.0f, w2 = v1 ? a2 * a2 : 0.0f, w3 = v1 ? a3 * a3 : 0.0f;
            l0 += w0 + w2;
            l1 += w1 + w3;
            constexpr float ps = (DT == EMBLA_F16) ? 0.015625f : 1.0f;
            pw[0] = w0 * ps;
            pw[1] = w1 * ps;
            pw[2] = w2 * ps;
            pw[3] = w3 * ps;
        } else {
            s[0] = v0 ? s[0] * scale : NEG_BIG;
            s[1] = v0 ? s[1] * scale : NEG_BIG;
            s[2] = v1 ? s[2] * scale : NEG_BIG;
            s[3] = v1 ? s[3] * scale : NEG_BIG;
            float tm0 = fmaxf(s[0], s[2]), tm1 = fmaxf(s[1], s[3]);
#pragma unroll
            for (int o = 4; o < 32; o <<= 1) {
                tm0 = fmaxf(tm0, __shfl_xor_sync(0xffffffffu, tm0, o));
                tm1 = fmaxf(tm1, __shfl_xor_sync(0xffffffffu, tm1, o));
            }
            const float n0 = fmaxf(m0, tm0), n1 = fmaxf(m1, tm1);
            const float f0 = __expf(m0 - n0), f1 = __expf(m1 - n1);
            m0 = n0;
            m1 = n1;
            pw[0] = v0 ? __expf(s[0] - m0) : 0.0f;
            pw[1] = v0 ? __expf(s[1] - m1) : 0.0f;
            pw[2] = v1 ? __expf(s[2] - m0) : 0.0f;
            pw[3] = v1 ? __expf(s[3] - m1) : 0.0f;
            l0 = l0 * f0 + pw[0] + pw[2];
            l1 = l1 * f1 + pw[1] + pw[3];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                OT[i][0] *= f0;
                OT[i][1] *= f1;
                OT[i][2] *= f0;
                OT[i][3] *= f1;
            }
        }
        const uint8_t* vA = Vt + (R0 + kA) * 128 + ((g ^ kA) << 4);
        const uint8_t* vB = Vt + (R0 + kB) * 128 + ((g ^ kB) << 4);
        uint4 A[2], B[2], C[2], D[2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            A[h] = *reinterpret_cast<const uint4*>(vA + h * (A16_ROWS * 128));
            B[h] = *reinterpret_cast<const uint4*>(vB + h * (A16_ROWS * 128));
            C[h] = *reinterpret_cast<const uint4*>(vA + h * (A16_ROWS * 128) + 8 * 128);
            D[h] = *reinterpret_cast<const uint4*>(vB + h * (A16_ROWS * 128) + 8 * 128);
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
        if (TMA) {
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[st]);   // this warp is done with the stage
        } else {
            cons_sync();   // every warp is done with this stage: the tile STAGES - 1 ahead may overwrite it
            if (t + A16_STAGES - 1 < ntile) issue_tile(t + A16_STAGES - 1);
            asm volatile("cp.async.commit_group;" ::: "memory");
            if (MODE == A16_SLIDING) {
                resolve_tile(t + A16_STAGES);
            } else {
                make_offsets();                      // tile t + STAGES, from the blocks looked up an iteration ago
                load_blocks();                       // tile t + STAGES + 1, from the index rows loaded an iteration ago
                load_rows(t + A16_STAGES + 2);       // their loads fly during the next tile's wait and compute
            }
        }
    }
    trace_last(p.ctl.trace, 2);
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
        l0 += __shfl_xor_sync(0xffffffffu, l0, o);
        l1 += __shfl_xor_sync(0xffffffffu, l1, o);
    }
    if (!TMA) asm volatile("cp.async.wait_group 0;" ::: "memory");
    cons_sync();   // every consumer is past its last tile: the stages are free
    if (TMA && *reinterpret_cast<volatile int*>(&s_failed)) {
        // a wait gave up: once the producer has stopped, wait (bounded) for the copies still on their way into the stages
        asm volatile("bar.sync 2, %0;" ::"n"(A16_THREADS + 32) : "memory");
        if (tid == 0) {
            const int issued = *reinterpret_cast<volatile int*>(&s_issued);
            for (int i = max(0, issued - A16_STAGES); i < issued; i++)
                if (!mbar_wait_bounded(p.ctl.wait_cycles, &full[i % A16_STAGES], (i / A16_STAGES) & 1)) atomicExch(p.ctl.err, ERR_WAIT_DRAIN);
        }
        cons_sync();
    }

    // ---- merge the 4 warps (in stage 0)
    float(*red)[8][HD] = reinterpret_cast<float(*)[8][HD]>(smem);
    float(*redm)[8] = reinterpret_cast<float(*)[8]>(smem + 4 * 8 * HD * 4);
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
    cons_sync();
    const int pair = b * p.n_kv_heads + kvh;
    // This CTA's merged partial goes to the global scratch or, with clusters, head by head into the inbox of the CTA that
    // finishes that head (head h: CTA h % nch), written straight into that CTA's shared memory.
    float* part = p.partials + (size_t(pair) * p.max_chunks + chunk) * p.G * A16_PART;
    float* inbox = reinterpret_cast<float*>(smem + A16_STAGES * A16_STAGE + 8 * HD * 2);
    const int slots = CL ? (p.G + nch - 1) / nch : 0;   // heads an owner finishes
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
            Act<DT>::store(p.o, size_t(b) * p.o_stride + size_t(kvh * p.G + hh) * HD + d, a16_finish<DT, MODE>(num, L));
        } else if (CL) {
            const uint32_t row = cluster_map(smem_u32(inbox + (chunk * slots + hh / nch) * A16_PART), uint32_t(hh % nch));
            cluster_st_f32(row + uint32_t(d) * 4u, num);
            if (d == 0) {
                cluster_st_f32(row + HD * 4, M);
                cluster_st_f32(row + (HD + 1) * 4, L);
            }
        } else {
            part[hh * A16_PART + d] = num;
            if (d == 0) {
                part[hh * A16_PART + HD] = M;
                part[hh * A16_PART + HD + 1] = L;
            }
        }
    }
    if (CL && nch > 1) {
        // One cluster barrier: every range's rows have arrived in their owners' inboxes; CTA `chunk` merges heads
        // chunk, chunk + nch, ... in range order from its own shared memory. Nobody touches another CTA's memory after the
        // barrier, so a CTA may leave as soon as it is done.
        cluster_arrive();
        cluster_wait();
        for (int slot = 0, hh = chunk; hh < p.G; slot++, hh += nch) {
            const int d = tid;
            float mc[8], lc[8], ac[8];
#pragma unroll
            for (int r = 0; r < 8; r++) {
                const float* row = inbox + ((r < nch ? r : 0) * slots + slot) * A16_PART;
                mc[r] = r < nch ? row[HD] : NEG_BIG;
                lc[r] = r < nch ? row[HD + 1] : 0.0f;
                ac[r] = r < nch ? row[d] : 0.0f;
            }
            float M = NEG_BIG;
#pragma unroll
            for (int r = 0; r < 8; r++) M = fmaxf(M, mc[r]);
            float L = 0.0f, num = 0.0f;
#pragma unroll
            for (int r = 0; r < 8; r++) {
                const float f = __expf(mc[r] - M);
                L += lc[r] * f;
                num += ac[r] * f;
            }
            Act<DT>::store(p.o, size_t(b) * p.o_stride + size_t(kvh * p.G + hh) * HD + d, a16_finish<DT, MODE>(num, L));
        }
        trace_last(p.ctl.trace, 3);
        return;
    }
    if (nch == 1) {
        trace_last(p.ctl.trace, 3);
        return;
    }
    __threadfence();
    cons_sync();
    if (tid == 0) {
        const int prev = atomicAdd(&p.counters[pair], 1);
        s_last = prev == nch - 1;
        if (s_last) p.counters[pair] = 0;
    }
    cons_sync();
    if (!s_last) {
        trace_last(p.ctl.trace, 3);
        return;
    }
    __threadfence();
    // the pair's partials (contiguous: [range][head][128 sums, max, sum]) into the free stages in one batch of loads,
    // then the merge in range order from shared memory
    const float* gbase = p.partials + size_t(pair) * p.max_chunks * p.G * A16_PART;
    float* sbase = reinterpret_cast<float*>(smem);
    stage_from_global<A16_THREADS>(reinterpret_cast<float4*>(sbase), reinterpret_cast<const float4*>(gbase), nch * p.G * (A16_PART / 4), tid);
    cons_sync();
    for (int idx = tid; idx < p.G * HD; idx += A16_THREADS) {
        const int hh = idx >> 7, d = idx & 127;
        float M = NEG_BIG;
        for (int cc = 0; cc < nch; cc++) M = fmaxf(M, sbase[(cc * p.G + hh) * A16_PART + HD]);
        float L = 0.0f, num = 0.0f;
        for (int cc = 0; cc < nch; cc++) {
            const float* q2 = sbase + (cc * p.G + hh) * A16_PART;
            const float f = __expf(q2[HD] - M);
            L += q2[HD + 1] * f;
            num += q2[d] * f;
        }
        Act<DT>::store(p.o, size_t(b) * p.o_stride + size_t(kvh * p.G + hh) * HD + d, a16_finish<DT, MODE>(num, L));
    }
    trace_last(p.ctl.trace, 3);
}

}  // namespace embla
