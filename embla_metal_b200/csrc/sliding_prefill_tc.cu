// Prefill-chunk attention of the sliding layers on the tensor cores (rings of a multiple of 128
// slots): every new token attends its last `window` positions, all already in the ring. Replaces attn_sliding_b /
// attn_sliding8_b (Sources/EmblaMetal/Kernels/prefill.metal:129-180, 439-548) for whole chunks; short chunks
// and odd rings take the mma.sync kernel of sliding_prefill.cu.
//
//   S = Q Kᵀ   tcgen05.mma kind::f16, M = 128 query rows, N = 128 keys (one 128-slot block of the ring), K = 128 dims
//   O += P V   A = P read from TMEM, B = V from shared memory (MN-major)
// A query tile is 128 / G consecutive tokens x the G query heads of one kv head (row = token * G + head), so all its
// rows share one run of ring blocks: the union of their windows, window + 128 / G - 1 positions. One CTA owns two
// consecutive tiles, which share every block fetched. The keys and values are 16-bit already: the TMA producer puts
// each block straight into the UMMA operand layout ([dims 0-63 | 64-127][128 keys][128 B], 128-byte swizzle), K as the
// K-major operand of Q Kᵀ and V as the MN-major operand of P V; no conversion warps.
//
// The softmax takes two passes over the blocks instead of rescaling O in TMEM: pass A runs only S = Q Kᵀ and the
// softmax warps keep each row's maximum over its window; pass B runs S again, p = exp(s - max) (masked to the row's own
// window), P in the activation dtype over the consumed S columns (bfloat16: P = hi + lo, two products, so that its
// rounding stays below 2^-16), O += P V; at the end O / Σp. A window is at most ten blocks, so
// the second Q Kᵀ costs half as much again as one pass and keeps the tensor pipe's work free of read-modify-write on O.
//   warps 0-7   two warpgroups, one per tile, one query row a thread
//   warp 8      TMA producer (3 buffers of 32 KiB: K blocks in pass A, K and V blocks in pass B)
//   warp 9      MMA issuer; in pass B per block S0, P V1 (block before), S1, P V0, as the full-layer kernel
// Every wait is bounded; a wait that runs out sets the context's error word and the CTA winds down.
#include "attn16_common.cuh"
#include "sliding_prefill_tc.cuh"
#include "tc05.cuh"

namespace embla {

constexpr int ST_PRODUCER = 8, ST_MMA = 9;
constexpr int ST_THREADS = (ST_MMA + 1) * 32;
constexpr int ST_TILE = BLK * HD * 2;     // 32 KiB
constexpr int ST_BUFS = 3;
constexpr size_t ST_SMEM = 1024 + 2 * ST_TILE + ST_BUFS * ST_TILE + 256;


template <int DT>
__global__ void __launch_bounds__(ST_THREADS, 1)
    sliding_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const SlidingTcParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* Qs = smem;                                  // [2 tiles][32 KiB]
    uint8_t* kvb = smem + 2 * ST_TILE;                   // [3][32 KiB] K or V blocks
    uint64_t* bars = reinterpret_cast<uint64_t*>(kvb + ST_BUFS * ST_TILE);
    uint64_t* kv_ready = bars;          // [3]
    uint64_t* kv_free = bars + 3;       // [3]
    uint64_t* s_full = bars + 6;        // [2 tiles]
    uint64_t* p_ready = bars + 8;       // [2 tiles]: the tile's warps are done with S (pass A) / have stored P (pass B)
    uint64_t* o_done = bars + 10;
    uint64_t* v_clean = bars + 11;      // the last V block holds no rows past the chunk any more
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kvh = blockIdx.y, b = blockIdx.z;
    const int tpt = BLK / p.G;                            // tokens of a tile
    const int p0 = p.pos0[b];
    int t0[2], ntok[2], jlo[2], jhi[2];
#pragma unroll
    for (int x = 0; x < 2; x++) {
        t0[x] = (2 * blockIdx.x + x) * tpt;
        ntok[x] = max(0, min(tpt, p.n_tokens - t0[x]));
        const int pa = p0 + t0[x], pz = pa + ntok[x] - 1;
        jlo[x] = max(0, pa - p.window + 1) >> 7;          // blocks of 128 positions the tile's windows touch
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

    if (tid == 0) {
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
    if (warp == ST_MMA) tmem_alloc(&s_tmem, 512);

    // ---- Q tiles: row r = token r / G, head r % G, as fp16 in the K-major swizzled layout (norm + RoPE at the token's
    // position when the queries arrive raw, as attn_sliding_b does)
    for (int x = 0; x < 2; x++) {
        uint8_t* Qx = Qs + x * ST_TILE;
        if (p.prenormed) {
            // rows as they are: 16 bytes a thread and trip, many loads in flight
#pragma unroll 4
            for (int i = tid; i < BLK * 16; i += ST_THREADS) {
                const int r = i >> 4, c8 = i & 15, t = r / p.G, hh = r % p.G;
                uint4 v = make_uint4(0, 0, 0, 0);
                if (t < ntok[x]) {
                    const size_t off = size_t(b) * p.q_seq_stride + size_t(t0[x] + t) * p.q_token_stride + size_t(kvh * p.G + hh) * HD + c8 * 8;
                    v = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.q) + off);
                }
                *reinterpret_cast<uint4*>(Qx + (c8 >> 3) * (BLK * 128) + r * 128 + (((c8 & 7) ^ (r & 7)) << 4)) = v;
            }
            continue;
        }
        // raw queries: four rows a warp and trip, their loads in flight together before the norms
        for (int r4 = warp * 4; r4 < BLK; r4 += 4 * (ST_THREADS / 32)) {
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
    fence_proxy_async();      // Q was written by ordinary stores; the tensor pipe reads it through the async proxy
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    // TMEM columns: S/P of tile 0 at 0, of tile 1 at 128 (P overwrites the first 64 columns of its S); O at 256, 384

    // Loads, in order: pass A the K block of every j; pass B the K block then the V block of every j. Load c uses buffer c % 3.
    if (warp == ST_PRODUCER) {
        if (lane == 0) {
            for (int c = 0; c < 3 * nblk; c++) {
                const int j = jb + (c < nblk ? c : (c - nblk) >> 1);
                const bool is_v = c >= nblk && ((c - nblk) & 1);
                const int slot = c % ST_BUFS;
                if (c >= ST_BUFS && !mbar_wait_bounded(p.ctl.wait_cycles, &kv_free[slot], ((c / ST_BUFS) - 1) & 1)) {
                    atomicCAS(p.ctl.err, 0, 1000 + c);
                    break;
                }
                if (*reinterpret_cast<volatile int*>(&s_abort)) break;
                const int y = kvh * p.ring + (j * BLK) % p.ring;
                uint8_t* dst = kvb + slot * ST_TILE;
                mbar_expect_tx(&kv_ready[slot], ST_TILE);
                tma_load_3d(dst, is_v ? &map_v : &map_k, 0, y, b, &kv_ready[slot]);
                tma_load_3d(dst + BLK * 128, is_v ? &map_v : &map_k, 128, y, b, &kv_ready[slot]);
            }
        }
        if (clean_v) {
            __syncwarp();
            const int cl = 3 * nblk - 1;                   // the last load: V of block je
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
            int c = 0;                 // loads consumed so far
            int site = 0;              // where a wait gave up: 100 pass + 10 step + ..., reported in the error word
            int us[2] = {0, 0};        // S products issued per tile (the phase counters of s_full / p_ready)
            auto wait_load = [&](int cc) {
                if (!mbar_wait_bounded(p.ctl.wait_cycles, &kv_ready[cc % ST_BUFS], (cc / ST_BUFS) & 1)) return false;
                return !(clean_v && cc == 3 * nblk - 1) || mbar_wait_bounded(p.ctl.wait_cycles, v_clean, 0);
            };
            // bfloat16 operands: formats of A and B in the instruction descriptor (bits 7-9 and 10-12)
            constexpr uint32_t fmt = DT == EMBLA_BF16 ? (1u << 7) | (1u << 10) : 0u;
            auto issue_s = [&](int x, int cc) {
                const uint32_t ka = smem_u32(kvb + (cc % ST_BUFS) * ST_TILE);
#pragma unroll
                for (int ks = 0; ks < 8; ks++) {
                    const uint32_t koff = (ks >> 2) * (BLK * 128) + (ks & 3) * 32;
                    umma_ss(tmem + 128 * x, umma_desc(qa + x * ST_TILE + koff, 16, 1024), umma_desc(ka + koff, 16, 1024), PF_IDESC_QK | fmt, ks > 0);
                }
                tc_commit(&s_full[x]);
                us[x]++;
            };
            auto issue_pv = [&](int x, int cc, bool first) {
                const uint32_t va = smem_u32(kvb + (cc % ST_BUFS) * ST_TILE);
#pragma unroll
                for (int ks = 0; ks < 8; ks++) {
                    const uint64_t vd = umma_desc(va + ks * 2048, BLK * 128, 1024);
                    if (DT == EMBLA_F16) {
                        umma_ts(tmem + 256 + 128 * x, tmem + 128 * x + 8 * ks, vd, PF_IDESC_PV, (!first) | (ks > 0));
                    } else {   // keys 64 h .. 64 h + 63: P hi at columns 64 h, P lo at 64 h + 32
                        const uint32_t pa = tmem + 128 * x + 64 * (ks >> 2) + 8 * (ks & 3);
                        umma_ts(tmem + 256 + 128 * x, pa, vd, PF_IDESC_PV | fmt, (!first) | (ks > 0));
                        umma_ts(tmem + 256 + 128 * x, pa + 32, vd, PF_IDESC_PV | fmt, 1);
                    }
                }
            };
            // the tile's warps are done with the S product before its us[x]-th (they arrive once per product)
            auto wait_tile = [&](int x) { return us[x] == 0 || mbar_wait_bounded(p.ctl.wait_cycles, &p_ready[x], (us[x] - 1) & 1); };
            // ---- pass A: row maxima
            for (int i = 0; i < nblk && ok; i++, c++) {
                const int j = jb + i;
                site = 100 + i;
                ok = wait_load(c);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int x = 0; x < 2; x++) {
                    if (j < jlo[x] || j > jhi[x]) continue;
                    site = 200 + 20 * x + i;
                    ok = ok && wait_tile(x);
                    if (!ok) break;
                    tc_fence_after();
                    issue_s(x, c);
                }
                tc_commit(&kv_free[c % ST_BUFS]);
            }
            // ---- pass B: S again, P V. Per block: S0, P V1 of the block before, S1, P V0.
            int pv1_load = -1;         // the V load of tile 1's pending P V
            bool first_pv[2] = {true, true};
            for (int i = 0; i <= nblk && ok; i++) {
                const int j = jb + i;
                const bool a0 = i < nblk && j >= jlo[0] && j <= jhi[0], a1 = i < nblk && j >= jlo[1] && j <= jhi[1];
                const int ck = c, cv = c + 1;
                if (i < nblk) {
                    site = 300 + i;
                    ok = wait_load(ck);
                    if (!ok) break;
                    tc_fence_after();
                }
                if (a0) {
                    site = 400 + i;
                    ok = wait_tile(0);      // pass A's last S of tile 0 has been read (first block), or P V0 before was issued
                    if (!ok) break;
                    tc_fence_after();
                    issue_s(0, ck);
                }
                if (pv1_load >= 0) {
                    site = 500 + i;
                    ok = mbar_wait_bounded(p.ctl.wait_cycles, &p_ready[1], (us[1] - 1) & 1) && wait_load(pv1_load);
                    if (!ok) break;
                    tc_fence_after();
                    issue_pv(1, pv1_load, first_pv[1]);
                    first_pv[1] = false;
                    tc_commit(&kv_free[pv1_load % ST_BUFS]);   // V of the block before: both tiles' P V are issued
                    pv1_load = -1;
                } else if (i >= 1) {
                    tc_commit(&kv_free[(c - 1) % ST_BUFS]);    // (tile 1 did not use that V)
                }
                if (a1) {
                    if (first_pv[1]) {       // pass A's last S of tile 1 must have been read before this overwrites it
                        site = 600 + i;
                        ok = wait_tile(1);
                        if (!ok) break;
                        tc_fence_after();
                    }
                    issue_s(1, ck);
                }
                if (i < nblk) tc_commit(&kv_free[ck % ST_BUFS]);   // K of this block
                if (a0) {
                    site = 700 + i;
                    ok = mbar_wait_bounded(p.ctl.wait_cycles, &p_ready[0], (us[0] - 1) & 1) && wait_load(cv);
                    if (!ok) break;
                    tc_fence_after();
                    issue_pv(0, cv, first_pv[0]);
                    first_pv[0] = false;
                }
                if (a1) pv1_load = cv;
                if (i < nblk) c += 2;
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
        const uint32_t tS = tmem + 128 * x, tO = tmem + 256 + 128 * x;
        const int tok = r / p.G;
        const bool row_ok = tok < ntok[x];
        const int pos_r = p0 + t0[x] + tok;                   // this row's position; it sees pos_r - window + 1 .. pos_r
        const int nx = ntok[x] > 0 ? jhi[x] - jlo[x] + 1 : 0;
        const float c2 = rsqrtf(float(HD)) * 1.4426950408889634f;   // scores to base-2 exponents
        float mrow = NEG_BIG, rowsum = 0.0f;
        bool ok = true;
        int u = 0;                                             // S products of this tile seen so far
        for (int pass = 0; pass < 2 && ok; pass++) {
            const float mc = mrow * c2;
            for (int i = 0; i < nx && ok; i++, u++) {
                const int j = jlo[x] + i;
                ok = __all_sync(0xffffffffu, mbar_wait_bounded(p.ctl.wait_cycles, &s_full[x], u & 1));
                if (!ok) break;   // (warp-uniform: the TMEM loads below are warp-collective)
                tc_fence_after();
                // weights of 32 keys from kb on: exp(s - max) masked to the row's window, summed in fp32, packed in pairs
                auto weights = [&](const uint32_t (&sv)[32], int kb, uint32_t (&hi)[16], uint32_t (&lo)[16]) {
#pragma unroll
                    for (int e = 0; e < 32; e += 2) {
                        const int kp = kb + e;
                        float w0 = exp2f(fmaf(__uint_as_float(sv[e]), c2, -mc)), w1 = exp2f(fmaf(__uint_as_float(sv[e + 1]), c2, -mc));
                        if (!(row_ok && kp <= pos_r && kp > pos_r - p.window)) w0 = 0.0f;
                        if (!(row_ok && kp + 1 <= pos_r && kp + 1 > pos_r - p.window)) w1 = 0.0f;
                        rowsum += w0 + w1;
                        hi[e >> 1] = pack_act2<DT>(w0, w1);
                        if (DT == EMBLA_BF16) lo[e >> 1] = pack_act2<DT>(w0 - Act<EMBLA_BF16>::round(w0), w1 - Act<EMBLA_BF16>::round(w1));
                    }
                };
                if (pass == 0) {
#pragma unroll
                    for (int cc = 0; cc < 4; cc++) {
                        uint32_t s[32];
                        tmem_ld32(tS + 32 * cc + lane_sel, s);
                        const int kb = j * BLK + 32 * cc;
#pragma unroll
                        for (int e = 0; e < 32; e++) {
                            const int kp = kb + e;
                            if (kp <= pos_r && kp > pos_r - p.window) mrow = fmaxf(mrow, __uint_as_float(s[e]));
                        }
                    }
                } else if (DT == EMBLA_F16) {
#pragma unroll
                    for (int cc = 0; cc < 4; cc++) {
                        uint32_t s[32], pk[16], unused[16];
                        tmem_ld32(tS + 32 * cc + lane_sel, s);
                        weights(s, j * BLK + 32 * cc, pk, unused);
                        // P goes over the S columns already consumed: chunk cc's 16 columns lie inside [0, 32 cc + 32)
                        tmem_st16(tS + 16 * cc + lane_sel, pk);
                    }
                } else {
                    // bfloat16: per 64 keys both S chunks are read before P hi (32 columns) and P lo (32 columns) overwrite them
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        uint32_t sa[32], ha[16], la[16];
                        tmem_ld32(tS + 64 * h + lane_sel, sa);
                        weights(sa, j * BLK + 64 * h, ha, la);
                        uint32_t sb[32], hb[16], lb[16];
                        tmem_ld32(tS + 64 * h + 32 + lane_sel, sb);
                        tmem_st16(tS + 64 * h + lane_sel, ha);
                        tmem_st16(tS + 64 * h + 32 + lane_sel, la);
                        weights(sb, j * BLK + 64 * h + 32, hb, lb);
                        tmem_st16(tS + 64 * h + 16 + lane_sel, hb);
                        tmem_st16(tS + 64 * h + 48 + lane_sel, lb);
                    }
                }
                if (pass == 1) tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&p_ready[x]);
            }
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
            // (the TMEM loads are warp-collective: every thread of the warpgroup takes them, rows past the chunk only skip the stores)
            tc_fence_after();
            const float inv = row_ok ? 1.0f / rowsum : 0.0f;
            uint16_t* orow = static_cast<uint16_t*>(p.o) + size_t(b) * p.o_seq_stride + size_t(t0[x] + tok) * p.o_token_stride +
                             size_t(kvh * p.G + r % p.G) * HD;
#pragma unroll 1
            for (int cc = 0; cc < 4; cc++) {
                uint32_t acc[32];
                tmem_ld32(tO + 32 * cc + lane_sel, acc);
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
