// Prefill-chunk attention of the sliding layers on the tensor cores (rings of a multiple of 128
// slots): every new token attends its last `window` positions, all already in the ring. Replaces attn_sliding_b /
// attn_sliding8_b (Sources/EmblaMetal/Kernels/prefill.metal:129-180, 439-548) for whole chunks; short chunks
// and odd rings take the mma.sync kernel of sliding_prefill.cu.
//
//   S = Q Kᵀ   tcgen05.mma kind::f16, M = 128 query rows, N = up to 128 keys (one 128-slot block of the ring), K = 128 dims
//   O += P V   A = P read from TMEM, B = V from shared memory (MN-major)
// A query tile is 128 / G consecutive tokens x the G query heads of one kv head (row = token * G + head), so all its
// rows share one run of ring blocks: the union of their windows, window + 128 / G - 1 positions. One CTA owns two
// consecutive tiles, which share every block fetched. The keys and values are 16-bit already: the TMA producer puts
// each block straight into the UMMA operand layout ([dims 0-63 | 64-127][128 keys][128 B], 128-byte swizzle), K as the
// K-major operand of Q Kᵀ and V as the MN-major operand of P V; no conversion warps. Of a block at the edge of a tile's
// windows only the 16-key groups some row can see are multiplied (N of Q Kᵀ and the k-steps of P V shrink to them).
//
// One pass over the blocks with a running row maximum that is allowed to go stale: p = exp2(s - m) where m is the
// maximum the row had when it was last adopted; m moves (and the row of O in TMEM and the row sum are rescaled by
// exp2(m_old - m_new)) only when a block's maximum exceeds it by more than 2^8, so p stays below 2^8, O and the sum
// share one m at all times, and O / Σp does not depend on it. After the first block or two a rescale is rare.
//   warps 0-7   two warpgroups, one per tile, one query row a thread: the row's 128 scores of a block are read into
//               registers at once (so P can go anywhere over S), maximum, weights, P; about four instructions a score
//   warp 8      TMA producer (4 buffers of 32 KiB: K block, V block, K block, ...)
//   warp 9      MMA issuer: per block P V of tile 0, S of tile 0 for the next block, P V of tile 1, S of tile 1 (next)
// A tile's next S is issued right behind its P V (the tensor pipe runs them in order), so the row's softmax of the next
// block overlaps the other tile's products. Every wait is bounded; a wait that runs out sets the context's error word
// and the CTA winds down.
#include "attn16_common.cuh"
#include "sliding_prefill_tc.cuh"
#include "tc05.cuh"

namespace embla {

constexpr int ST_SOFTMAX_WARPS = 8, ST_PRODUCER = 8, ST_MMA = 9;
constexpr int ST_THREADS = (ST_MMA + 1) * 32;
constexpr int ST_TILE = BLK * HD * 2;     // 32 KiB
constexpr int ST_BUFS = 4;
constexpr size_t ST_SMEM = 1024 + 2 * ST_TILE + ST_BUFS * ST_TILE + 256;
constexpr float ST_STALE = 8.0f;          // how far (in powers of two) a block's maximum may exceed the adopted one

// max of three (one instruction on this architecture)
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// The 16-key groups [n0, n1) of block j that hold a key of [klo, khi] (the union of a tile's windows); false if none.
__device__ __forceinline__ bool block_cols(int j, int jlo, int jhi, int klo, int khi, int& n0, int& n1) {
    if (j < jlo || j > jhi) return false;
    n0 = max(klo - j * BLK, 0) & ~15;
    n1 = (min(khi - j * BLK, BLK - 1) + 16) & ~15;
    return true;
}

template <int DT>
__global__ void __launch_bounds__(ST_THREADS, 1)
    sliding_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const SlidingTcParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* Qs = smem;                                  // [2 tiles][32 KiB]
    uint8_t* kvb = smem + 2 * ST_TILE;                   // [4][32 KiB] K or V blocks
    uint64_t* bars = reinterpret_cast<uint64_t*>(kvb + ST_BUFS * ST_TILE);
    uint64_t* kv_ready = bars;          // [4]
    uint64_t* kv_free = bars + 4;       // [4]
    uint64_t* s_full = bars + 8;        // [2 tiles]
    uint64_t* p_ready = bars + 10;      // [2 tiles]: the tile's 4 warps have stored P
    uint64_t* o_done = bars + 14;
    uint64_t* v_clean = bars + 15;      // the last V block holds no rows past the chunk any more
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kvh = blockIdx.y, b = blockIdx.z;
    const int tpt = BLK / p.G;                            // tokens of a tile
    const int p0 = p.pos0[b];
    int t0[2], ntok[2], jlo[2], jhi[2], klo[2], khi[2];
#pragma unroll
    for (int x = 0; x < 2; x++) {
        t0[x] = (2 * blockIdx.x + x) * tpt;
        ntok[x] = max(0, min(tpt, p.n_tokens - t0[x]));
        const int pa = p0 + t0[x], pz = pa + ntok[x] - 1;
        klo[x] = max(0, pa - p.window + 1);               // the keys some row of the tile sees
        khi[x] = pz;
        jlo[x] = klo[x] >> 7;                             // blocks of 128 positions they lie in
        jhi[x] = ntok[x] > 0 ? pz >> 7 : -1;
    }
    const int jb = ntok[1] > 0 ? min(jlo[0], jlo[1]) : jlo[0];
    const int je = max(jhi[0], jhi[1]);
    const int nblk = je - jb + 1;                          // >= 1: tile 0 always has a token
    // Slots after the chunk's last position may never have been written (a sequence shorter than the ring): their keys
    // are masked, but their value rows would poison P V even with zero weights. They can only lie in the block of the
    // chunk's last position, which is then this CTA's last block: the producer zeroes those rows of the staged V.
    const int chunk_end = p0 + p.n_tokens - 1;
    const bool clean_v = je == (chunk_end >> 7) && (chunk_end & (BLK - 1)) != BLK - 1;

    // The producer sets the barriers up and requests the first blocks while the other warps stage Q.
    if (warp == ST_PRODUCER && lane == 0) {
        for (int i = 0; i < ST_BUFS; i++) {
            mbar_init(&kv_ready[i], 1);
            mbar_init(&kv_free[i], 1);
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(&s_full[i], 1);
            mbar_init(&p_ready[i], 4);
        }
        mbar_init(o_done, 1);
        mbar_init(v_clean, 1);
        s_abort = 0;
        fence_barrier_init();
    }
    auto request = [&](int c) {                            // load c: K of block jb + c / 2 (even c) or its V (odd c)
        const int j = jb + (c >> 1), slot = c % ST_BUFS;
        const int y = kvh * p.ring + (j * BLK) % p.ring;
        uint8_t* dst = kvb + slot * ST_TILE;
        const CUtensorMap* map = (c & 1) ? &map_v : &map_k;
        mbar_expect_tx(&kv_ready[slot], ST_TILE);
        tma_load_3d(dst, map, 0, y, b, &kv_ready[slot]);
        tma_load_3d(dst + BLK * 128, map, 128, y, b, &kv_ready[slot]);
    };
    if (warp == ST_PRODUCER && lane == 0)
        for (int c = 0; c < min(ST_BUFS, 2 * nblk); c++) request(c);
    if (warp == ST_MMA) tmem_alloc(&s_tmem, 512);

    // ---- Q tiles: row r = token r / G, head r % G, as fp16 in the K-major swizzled layout (norm + RoPE at the token's
    // position when the queries arrive raw, as attn_sliding_b does)
    if (warp < ST_SOFTMAX_WARPS && p.prenormed) {
        // rows as they are: 16 bytes a thread and trip, all sixteen loads of a thread (both tiles) in flight before the stores
        constexpr int TRIPS = BLK * 16 / (ST_SOFTMAX_WARPS * 32);
        uint4 v[2][TRIPS];
#pragma unroll
        for (int x = 0; x < 2; x++) {
#pragma unroll
            for (int k = 0; k < TRIPS; k++) {
                const int i = tid + k * (ST_SOFTMAX_WARPS * 32), r = i >> 4, c8 = i & 15, t = r / p.G, hh = r % p.G;
                v[x][k] = make_uint4(0, 0, 0, 0);
                if (t < ntok[x]) {
                    const size_t off = size_t(b) * p.q_seq_stride + size_t(t0[x] + t) * p.q_token_stride + size_t(kvh * p.G + hh) * HD + c8 * 8;
                    v[x][k] = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.q) + off);
                }
            }
        }
#pragma unroll
        for (int x = 0; x < 2; x++) {
#pragma unroll
            for (int k = 0; k < TRIPS; k++) {
                const int i = tid + k * (ST_SOFTMAX_WARPS * 32), r = i >> 4, c8 = i & 15;
                *reinterpret_cast<uint4*>(Qs + x * ST_TILE + (c8 >> 3) * (BLK * 128) + r * 128 + (((c8 & 7) ^ (r & 7)) << 4)) = v[x][k];
            }
        }
        fence_proxy_async();  // Q was written by ordinary stores; the tensor pipe reads it through the async proxy
    } else if (warp < ST_SOFTMAX_WARPS) {
        for (int x = 0; x < 2; x++) {
            uint8_t* Qx = Qs + x * ST_TILE;
            // raw queries: four rows a warp and trip, their loads in flight together before the norms
            for (int r4 = warp * 4; r4 < BLK; r4 += 4 * ST_SOFTMAX_WARPS) {
                float xq[4][4];
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const int r = r4 + k, t = r / p.G, hh = r % p.G;
                    const size_t off = size_t(b) * p.q_seq_stride + size_t(t0[x] + t) * p.q_token_stride + size_t(kvh * p.G + hh) * HD;
#pragma unroll
                    for (int i = 0; i < 4; i++) xq[k][i] = t < ntok[x] ? Act<DT>::load(p.q, off + lane + 32 * i) : 0.0f;
                }
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const int r = r4 + k, t = r / p.G;
                    if (t < ntok[x]) norm_rope_round<DT>(xq[k], p.g1, p.g1, 1, p0 + t0[x] + t, p.rope_freq, lane);
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const int d = lane + 32 * i, c8 = d >> 3;
                        Act<DT>::store(Qx + (c8 >> 3) * (BLK * 128) + r * 128 + (((c8 & 7) ^ (r & 7)) << 4) + (d & 7) * 2, 0, xq[k][i]);
                    }
                }
            }
        }
        fence_proxy_async();  // Q was written by ordinary stores; the tensor pipe reads it through the async proxy
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    // TMEM columns: S of tile 0 at 0, of tile 1 at 128; O at 256, 384. P of keys 64 h + 16 k .. + 15 goes over S: 8 columns
    // at 64 h + 8 k (bfloat16: its low part 32 columns further on).

    if (warp == ST_PRODUCER) {
        if (lane == 0) {
            for (int c = ST_BUFS; c < 2 * nblk; c++) {
                if (!mbar_wait_bounded(p.ctl.wait_cycles, &kv_free[c % ST_BUFS], ((c / ST_BUFS) - 1) & 1)) {
                    atomicCAS(p.ctl.err, 0, 1000 + c);
                    break;
                }
                if (*reinterpret_cast<volatile int*>(&s_abort)) break;
                request(c);
            }
        }
        if (clean_v) {
            __syncwarp();
            const int cl = 2 * nblk - 1;                   // the last load: V of block je
            uint8_t* vb = kvb + (cl % ST_BUFS) * ST_TILE;
            if (mbar_wait_bounded(p.ctl.wait_cycles, &kv_ready[cl % ST_BUFS], (cl / ST_BUFS) & 1)) {
                const int first = (chunk_end & (BLK - 1)) + 1;
                for (int i = first * 16 + lane; i < BLK * 16; i += 32) {      // 16 x 16 bytes a row: 8 in each half
                    const int row = i >> 4, q16 = i & 15;
                    *reinterpret_cast<uint4*>(vb + (q16 >> 3) * (BLK * 128) + row * 128 + (q16 & 7) * 16) = make_uint4(0, 0, 0, 0);
                }
                fence_proxy_async();
            } else if (lane == 0) {
                atomicCAS(p.ctl.err, 0, 1900);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(v_clean);
        }
    } else if (warp == ST_MMA) {
        if (lane == 0) {
            const uint32_t qa = smem_u32(Qs);
            bool ok = true;
            int site = 0;              // where a wait gave up, reported in the error word
            int us[2] = {0, 0};        // S products issued per tile (the phase counters of s_full / p_ready)
            auto wait_load = [&](int cc) {
                if (!mbar_wait_bounded(p.ctl.wait_cycles, &kv_ready[cc % ST_BUFS], (cc / ST_BUFS) & 1)) return false;
                return !(clean_v && cc == 2 * nblk - 1) || mbar_wait_bounded(p.ctl.wait_cycles, v_clean, 0);
            };
            // bfloat16 operands: formats of A and B in the instruction descriptor (bits 7-9 and 10-12)
            constexpr uint32_t fmt = DT == EMBLA_BF16 ? (1u << 7) | (1u << 10) : 0u;
            auto issue_s = [&](int x, int cc, int n0, int n1) {       // keys n0 .. n1 - 1 of the block in buffer cc % 4
                const uint32_t ka = smem_u32(kvb + (cc % ST_BUFS) * ST_TILE) + n0 * 128;
                const uint32_t idesc = ((PF_IDESC_QK & ~(0x3Fu << 17)) | (uint32_t(n1 - n0) >> 3 << 17)) | fmt;
#pragma unroll
                for (int ks = 0; ks < 8; ks++) {
                    const uint32_t koff = (ks >> 2) * (BLK * 128) + (ks & 3) * 32;
                    umma_ss(tmem + 128 * x + n0, umma_desc(qa + x * ST_TILE + koff, 16, 1024), umma_desc(ka + koff, 16, 1024), idesc, ks > 0);
                }
                tc_commit(&s_full[x]);
                us[x]++;
            };
            auto issue_pv = [&](int x, int cc, bool first, int n0, int n1) {
                const uint32_t va = smem_u32(kvb + (cc % ST_BUFS) * ST_TILE);
                for (int ks = n0 >> 4; ks < n1 >> 4; ks++) {
                    const uint64_t vd = umma_desc(va + ks * 2048, BLK * 128, 1024);
                    const uint32_t pa = tmem + 128 * x + 64 * (ks >> 2) + 8 * (ks & 3);
                    umma_ts(tmem + 256 + 128 * x, pa, vd, PF_IDESC_PV | fmt, (!first) | (ks > (n0 >> 4)));
                    if (DT == EMBLA_BF16) umma_ts(tmem + 256 + 128 * x, pa + 32, vd, PF_IDESC_PV | fmt, 1);
                }
            };
            int n0 = 0, n1 = 0;
            // ---- the first block's S products
            site = 100;
            ok = wait_load(0);
            if (ok) {
                tc_fence_after();
#pragma unroll
                for (int x = 0; x < 2; x++)
                    if (block_cols(jb, jlo[x], jhi[x], klo[x], khi[x], n0, n1)) issue_s(x, 0, n0, n1);
                tc_commit(&kv_free[0]);
            }
            // ---- per block: P V of tile 0, S of tile 0 on the next block, P V of tile 1, S of tile 1 on the next block
            bool first_pv[2] = {true, true};
            for (int i = 0; i < nblk && ok; i++) {
                const int j = jb + i, cv = 2 * i + 1, ck = 2 * i + 2;
                const bool next = i + 1 < nblk;
                bool k_here = false;
                site = 200 + i;
                ok = wait_load(cv);
                if (!ok) break;
#pragma unroll
                for (int x = 0; x < 2; x++) {
                    if (block_cols(j, jlo[x], jhi[x], klo[x], khi[x], n0, n1)) {
                        site = 300 + 100 * x + i;
                        ok = mbar_wait_bounded(p.ctl.wait_cycles, &p_ready[x], (us[x] - 1) & 1);
                        if (!ok) break;
                        tc_fence_after();
                        issue_pv(x, cv, first_pv[x], n0, n1);
                        first_pv[x] = false;
                    }
                    if (x == 1) tc_commit(&kv_free[cv % ST_BUFS]);     // V of this block: both tiles' P V are issued
                    if (next && block_cols(j + 1, jlo[x], jhi[x], klo[x], khi[x], n0, n1)) {
                        if (!k_here) {
                            site = 500 + i;
                            ok = wait_load(ck);
                            if (!ok) break;
                            tc_fence_after();
                            k_here = true;
                        }
                        issue_s(x, ck, n0, n1);
                    }
                }
                if (next && ok) tc_commit(&kv_free[ck % ST_BUFS]);     // K of the next block: both tiles' S are issued
            }
            if (!ok) {
                atomicCAS(p.ctl.err, 0, 2000 + site);
                *reinterpret_cast<volatile int*>(&s_abort) = 1;
            }
            tc_commit(o_done);
        }
    } else {
        // ---- softmax warps: warpgroup x owns tile x, one query row a thread
        const int x = warp >> 2, r = tid & 127;
        const uint32_t lane_sel = uint32_t((warp & 3) * 32) << 16;
        const uint32_t tS = tmem + 128 * x + lane_sel, tO = tmem + 256 + 128 * x + lane_sel;
        const int tok = r / p.G;
        const bool row_ok = tok < ntok[x];
        const int pos_r = p0 + t0[x] + tok;                   // this row's position; it sees pos_r - window + 1 .. pos_r
        const int nx = ntok[x] > 0 ? jhi[x] - jlo[x] + 1 : 0;
        const float c2 = rsqrtf(float(HD)) * 1.4426950408889634f;   // scores to base-2 exponents
        float m2 = NEG_BIG, rowsum = 0.0f;                    // adopted maximum (base-2 exponent), sum of the weights
        bool ok = true;
        int u = 0;                                             // S products of this tile seen so far
        for (; u < nx && ok; u++) {
            const int j = jlo[x] + u;
            int n0 = 0, n1 = 0;
            block_cols(j, jlo[x], jhi[x], klo[x], khi[x], n0, n1);
            // visible keys of this row in the block: lo_r <= e <= hi_r
            const int lo_r = row_ok ? pos_r - p.window + 1 - j * BLK : BLK, hi_r = pos_r - j * BLK;
            // a chunk of 32 keys is taken if it holds a key of the tile's windows, and needs no masks if every row of a
            // full tile sees all its keys (both the same for the whole tile)
            bool act[4], inner[4];
#pragma unroll
            for (int cc = 0; cc < 4; cc++) {
                act[cc] = 32 * cc < n1 && 32 * cc + 32 > n0;
                inner[cc] = ntok[x] == tpt && j * BLK + 32 * cc + 31 <= p0 + t0[x] && j * BLK + 32 * cc >= khi[x] - p.window + 1;
            }
            ok = __all_sync(0xffffffffu, mbar_wait_bounded(p.ctl.wait_cycles, &s_full[x], u & 1));
            if (!ok) break;   // (warp-uniform: the TMEM loads below are warp-collective)
            tc_fence_after();
            uint32_t s[4][32];
#pragma unroll
            for (int cc = 0; cc < 4; cc++)
                if (act[cc]) tmem_ld32_async(tS + 32 * cc, s[cc]);
            float bm = NEG_BIG;
#pragma unroll
            for (int cc = 0; cc < 4; cc++) {
                if (!act[cc]) continue;
                tmem_ld_arrived(s[cc]);
                if (inner[cc]) {
#pragma unroll
                    for (int e = 0; e < 32; e += 2) bm = max3(bm, __uint_as_float(s[cc][e]), __uint_as_float(s[cc][e + 1]));
                } else {
#pragma unroll
                    for (int e = 0; e < 32; e++)
                        if (32 * cc + e >= lo_r && 32 * cc + e <= hi_r) bm = fmaxf(bm, __uint_as_float(s[cc][e]));
                }
            }
            const float bm2 = bm * c2;
            if (u == 0) {
                m2 = bm2;                                      // nothing accumulated yet
            } else if (__any_sync(0xffffffffu, bm2 > m2 + ST_STALE)) {
                // (the tile's S of this block is complete, so its P V of the block before is: O is at rest)
                const float mn = fmaxf(m2, bm2), f = ex2_approx(m2 - mn);
                m2 = mn;
                rowsum *= f;
#pragma unroll 1
                for (int cc = 0; cc < 4; cc++) {
                    uint32_t acc[32];
                    tmem_ld32(tO + 32 * cc, acc);
#pragma unroll
                    for (int e = 0; e < 32; e++) acc[e] = __float_as_uint(__uint_as_float(acc[e]) * f);
                    tmem_st32(tO + 32 * cc, acc);
                }
            }
            // weights of a chunk: exp2(s - m), masked to the row's window where the chunk needs it, summed in fp32, packed in pairs
            const float nm2 = -m2;
#pragma unroll
            for (int cc = 0; cc < 4; cc++) {
                if (!act[cc]) continue;
                uint32_t hi[16], lo[16];
                float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
                for (int e = 0; e < 32; e += 2) {
                    float w0 = ex2_approx(fmaf(__uint_as_float(s[cc][e]), c2, nm2)), w1 = ex2_approx(fmaf(__uint_as_float(s[cc][e + 1]), c2, nm2));
                    if (!inner[cc]) {
                        if (!(32 * cc + e >= lo_r && 32 * cc + e <= hi_r)) w0 = 0.0f;
                        if (!(32 * cc + e + 1 >= lo_r && 32 * cc + e + 1 <= hi_r)) w1 = 0.0f;
                    }
                    sum0 += w0;
                    sum1 += w1;
                    hi[e >> 1] = pack_act2<DT>(w0, w1);
                    if (DT == EMBLA_BF16) lo[e >> 1] = pack_act2<DT>(w0 - Act<EMBLA_BF16>::round(w0), w1 - Act<EMBLA_BF16>::round(w1));
                }
                rowsum += sum0 + sum1;
                tmem_st16(tS + 64 * (cc >> 1) + 16 * (cc & 1), hi);
                if (DT == EMBLA_BF16) tmem_st16(tS + 64 * (cc >> 1) + 16 * (cc & 1) + 32, lo);
            }
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_ready[x]);
        }
        if (ok) {
            ok = mbar_wait_bounded(p.ctl.wait_cycles, o_done, 0);
            if (!ok) u = 99;
        }
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
            atomicCAS(p.ctl.err, 0, 3000 + 100 * x + u);
            *reinterpret_cast<volatile int*>(&s_abort) = 1;
        } else if (ntok[x] > 0) {
            // (the TMEM loads are warp-collective: every thread of the warp takes them, rows past the chunk only skip the stores)
            tc_fence_after();
            const float inv = row_ok ? 1.0f / rowsum : 0.0f;
            uint16_t* orow = static_cast<uint16_t*>(p.o) + size_t(b) * p.o_seq_stride + size_t(t0[x] + tok) * p.o_token_stride +
                             size_t(kvh * p.G + r % p.G) * HD;
#pragma unroll 1
            for (int cc = 0; cc < 4; cc++) {
                uint32_t acc[32];
                tmem_ld32(tO + 32 * cc, acc);
                if (row_ok) {
                    uint32_t outw[16];
#pragma unroll
                    for (int e = 0; e < 32; e += 2) outw[e >> 1] = pack_act2<DT>(__uint_as_float(acc[e]) * inv, __uint_as_float(acc[e + 1]) * inv);
#pragma unroll
                    for (int v4 = 0; v4 < 4; v4++)
                        *reinterpret_cast<uint4*>(orow + 32 * cc + 8 * v4) = make_uint4(outw[4 * v4], outw[4 * v4 + 1], outw[4 * v4 + 2], outw[4 * v4 + 3]);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == ST_MMA) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

// Launch for the whole batch; the rings' tensor maps (boxes of 128 rows x 128 bytes) are encoded per call.
EmblaStatus launch_sliding_prefill_tc(EmblaAttn* ctx, const EmblaRing* ring, const SlidingTcParams& p, int batch, cudaStream_t s) {
    TensorMapEncodeTiledFn enc = tensor_map_encoder();
    if (!enc) EMBLA_FAIL(EMBLA_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    CUtensorMap mk, mv;
    const cuuint64_t dims[3] = {HD * 2, cuuint64_t(p.n_kv_heads) * p.ring, cuuint64_t(batch)};
    const cuuint64_t strides[2] = {HD * 2, cuuint64_t(ring->seq_stride) * 2};
    const cuuint32_t box[3] = {128, BLK, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    for (int side = 0; side < 2; side++) {
        CUresult r = enc(side ? &mv : &mk, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, side ? ring->v_dev : ring->k_dev, dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) EMBLA_FAIL(EMBLA_CUDA, "cuTensorMapEncodeTiled failed for a ring (%d)", int(r));
    }
    const bool bf = ctx->cfg.act_dtype == EMBLA_BF16;
    auto kern = bf ? sliding_prefill_tc_kernel<EMBLA_BF16> : sliding_prefill_tc_kernel<EMBLA_F16>;
    static bool configured[2][64] = {};
    if (!configured[bf][ctx->device & 63]) {
        EMBLA_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(ST_SMEM)));
        configured[bf][ctx->device & 63] = true;
    }
    const int tpt = BLK / p.G;
    dim3 grid((p.n_tokens + 2 * tpt - 1) / (2 * tpt), p.n_kv_heads, batch);
    kern<<<grid, ST_THREADS, ST_SMEM, s>>>(mk, mv, p);
    EMBLA_CUDA_TRY(cudaGetLastError());
    return EMBLA_OK;
}

}  // namespace embla
