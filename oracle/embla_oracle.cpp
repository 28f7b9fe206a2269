// TEST INFRASTRUCTURE — not part of the product.
//
// Scalar CPU restatement of the attention hot path of sevren-ai/embla-metal (Swift + Metal). The
// reference ships no CPU implementation of attention and nothing of it can be compiled off Apple
// hardware, so this file restates the arithmetic of its .metal kernels in plain C++ (a loop stands
// in for a simdgroup). It is the parity checker for the CUDA library and the timed CPU baseline;
// only tests, the smoke check and the bench's cpu_baseline / reference arm may load it.
//
// PARITY UNPINNED: the reference holds no golden vectors, known-answer tests or unit tests for
// attention, KV quantisation, key scoring or selection (Tests/ covers GEMV/GEMM/sampler/chat only).
// The only check the reference itself owns for this path is Engine.verifySelection
// (Sources/EmblaMetal/Engine.swift:1115-1131), restated here as orc_verify_selection.
//
// Conventions
//   * 16-bit activations are raw uint16 storage with a dtype flag: 0 = bfloat16, 1 = float16.
//     The reference is bfloat16 throughout; "round to the storage dtype" generalises its bf()
//     (Sources/EmblaMetal/Kernels/common.metal:13; rounding rule Sources/EmblaMetal/BFloat16.swift:4-8).
//   * All sums are fp32. The 128-term q·k dot is ONE fused-multiply-add chain over d = 0..127
//     starting from 0 (canon_dot). The reference sums 4 dims a lane and then simd_sum()s
//     (common.metal:28-29, attention.metal:184-188); Apple leaves simd_sum's order unspecified, so
//     a fixed order has to be chosen, and this one is what the CUDA scoring kernels reproduce
//     bit for bit so that top-k index sets can be compared exactly.
//   * Tensors are dense and layout-agnostic: K/V caches are [kv head][ldS rows][128].
//
// Build: see oracle/Makefile (g++ -O2 -ffp-contract=off, no intrinsics).

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>
#include <thread>
#include <vector>

namespace {

constexpr int HD = 128;                      // head dim (common.metal:7)
constexpr float EPS32 = 1.1920929e-07f;      // common.metal:9
constexpr float NEG = -1e30f;                // common.metal:10
constexpr int TOPK = 1024, RECENT = 128;     // attention.metal:655

// ---- storage dtypes ---------------------------------------------------------------------------
inline float bf16_to_f(uint16_t b) { uint32_t u = uint32_t(b) << 16; float f; std::memcpy(&f, &u, 4); return f; }
inline uint16_t f_to_bf16(float f) {   // round to nearest even, BFloat16.swift:4-8
    uint32_t u; std::memcpy(&u, &f, 4);
    const uint32_t rounding = ((u >> 16) & 1u) + 0x7FFFu;
    return uint16_t((u + rounding) >> 16);
}
inline float f16_to_f(uint16_t h) { _Float16 x; std::memcpy(&x, &h, 2); return float(x); }
inline uint16_t f_to_f16(float f) { _Float16 x = _Float16(f); uint16_t h; std::memcpy(&h, &x, 2); return h; }

inline float load_act(uint16_t s, int dtype) { return dtype == 0 ? bf16_to_f(s) : f16_to_f(s); }
inline uint16_t store_act(float f, int dtype) { return dtype == 0 ? f_to_bf16(f) : f_to_f16(f); }
inline float round_act(float f, int dtype) { return load_act(store_act(f, dtype), dtype); }

// ---- helpers of common.metal -------------------------------------------------------------------
// RMS norm of one head times the gains 1 + w of the first ng of g1, g2 (common.metal:30-41).
// The sum of squares is taken in the reference's lane order: lane l adds dims l, l+32, l+64, l+96,
// then the 32 lane sums are added in lane order.
void head_norm(float* v, const uint16_t* g1, const uint16_t* g2, int ng, int dtype) {
    float total = 0.0f;
    for (int l = 0; l < 32; l++) {
        float ss = 0.0f;
        for (int i = 0; i < 4; i++) ss += v[l + 32 * i] * v[l + 32 * i];
        total += ss;
    }
    const float r = 1.0f / std::sqrt(total / float(HD) + EPS32);
    for (int d = 0; d < HD; d++) {
        float g = r;
        if (ng >= 1) g *= 1.0f + load_act(g1[d], dtype);
        if (ng >= 2) g *= 1.0f + load_act(g2[d], dtype);
        v[d] *= g;
    }
}

// RoPE on the first 64 dims, pairs (l, l+32), by -theta (common.metal:45-51).
void rope(float* v, int pos) {
    for (int l = 0; l < 32; l++) {
        const float theta = -float(pos) * std::exp2(-float(l) / 32.0f * 13.287712379549449f);
        const float c = std::cos(theta), s = std::sin(theta);
        const float x1 = v[l], x2 = v[l + 32];
        v[l] = x1 * c - x2 * s;
        v[l + 32] = x1 * s + x2 * c;
    }
}

// The canonical 128-term dot: one fmaf chain over d ascending.
inline float canon_dot(const float* q, const float* k) {
    float acc = 0.0f;
    for (int d = 0; d < HD; d++) acc = std::fmaf(q[d], k[d], acc);
    return acc;
}

// The query of one head as the attention kernels use it: optional head norm (+ RoPE), then rounded
// to the storage dtype (attention.metal:47-54, 166-169). `prenormed` skips norm and RoPE.
void prep_q(const uint16_t* q, int dtype, int prenormed, const uint16_t* g1, const uint16_t* g2, int ng,
            int rope_pos, float* out) {
    for (int d = 0; d < HD; d++) out[d] = load_act(q[d], dtype);
    if (!prenormed) {
        head_norm(out, g1, g2, ng, dtype);
        if (rope_pos >= 0) rope(out, rope_pos);
        for (int d = 0; d < HD; d++) out[d] = round_act(out[d], dtype);
    }
}

// A cache row as fp32: int8 codes (scale applied by the caller) or 16-bit storage.
inline void load_row(const void* base, int kv_kind, int dtype, size_t row, float* out) {
    if (kv_kind == 0) {
        const int8_t* p = static_cast<const int8_t*>(base) + row * HD;
        for (int d = 0; d < HD; d++) out[d] = float(p[d]);
    } else {
        const uint16_t* p = static_cast<const uint16_t*>(base) + row * HD;
        for (int d = 0; d < HD; d++) out[d] = load_act(p[d], dtype);
    }
}

inline uint32_t order_bits(float f) {   // attention.metal:657-660
    uint32_t u; std::memcpy(&u, &f, 4);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

void parallel_for(int n, int nthreads, const std::function<void(int)>& fn) {
    if (nthreads <= 1 || n <= 1) { for (int i = 0; i < n; i++) fn(i); return; }
    std::vector<std::thread> pool;
    const int t = std::min(nthreads, n);
    for (int w = 0; w < t; w++) pool.emplace_back([=, &fn] { for (int i = w; i < n; i += t) fn(i); });
    for (auto& th : pool) th.join();
}

}  // namespace

extern "C" {

float orc_round_act(float x, int dtype) { return round_act(x, dtype); }
uint32_t orc_order_bits(float f) { return order_bits(f); }

// ---- quantised append --------------------------------------------------------------------------
// write_row8 (common.metal:74-84) for n rows: x rounded to the storage dtype, a = max|x|,
// code = rint(x * (127 / a)) (round half to even), scale = a / 127; a == 0 gives codes 0, scale 0.
// With `norm`, the row is first RMS-normed without gains, as kv_append does to keys
// (attention.metal:128). `scale_dtype`: 0 = fp32 (the reference), 1 = the scale rounded to fp16.
void orc_quantize_rows(const uint16_t* x, int n, int dtype, int norm, int scale_dtype, int8_t* codes, float* scales) {
    for (int r = 0; r < n; r++) {
        float v[HD];
        for (int d = 0; d < HD; d++) v[d] = load_act(x[size_t(r) * HD + d], dtype);
        if (norm) head_norm(v, nullptr, nullptr, 0, dtype);
        float a = 0.0f;
        for (int d = 0; d < HD; d++) { v[d] = round_act(v[d], dtype); a = std::max(a, std::fabs(v[d])); }
        const float inv = a > 0.0f ? 127.0f / a : 0.0f;
        for (int d = 0; d < HD; d++) codes[size_t(r) * HD + d] = int8_t(int(std::rint(v[d] * inv)));
        float s = a / 127.0f;
        if (scale_dtype == 1) s = f16_to_f(f_to_f16(s));
        scales[r] = s;
    }
}

// ---- full layers, decode (ReLU²) ---------------------------------------------------------------
// attn_full / attn_full8 (attention.metal:148-220, 235-363): t_j = q·k_j (· key scale for int8),
// w_j = max(t_j / sqrt(D), 0)², o = sum_j w_j v_j / (sqrt(D) + sum_j w_j), rounded to the storage
// dtype. With `scores`, scores[kvh][j] = max over the kv head's query heads of t_j, without the
// 1/sqrt(D) (attention.metal:189, 203-205, 295-303); ties keep the earlier head.
// kv_kind 0: int8 codes with per-row fp32 scales; 1: 16-bit rows in the storage dtype (scales unused).
void orc_full_decode(const uint16_t* q, int dtype, int prenormed, const uint16_t* g1, const uint16_t* g2, int ng,
                     int kv_kind, const void* kc, const float* ks, const void* vc, const float* vs,
                     int Hq, int Hkv, int S, int ldS, uint16_t* o, float* scores) {
    const int G = Hq / Hkv;
    const float scale = 1.0f / std::sqrt(float(HD));
    std::vector<float> qn(size_t(Hq) * HD);
    for (int h = 0; h < Hq; h++) prep_q(q + size_t(h) * HD, dtype, prenormed, g1, g2, ng, -1, &qn[size_t(h) * HD]);
    std::vector<float> acc(size_t(Hq) * HD, 0.0f), psum(Hq, 0.0f);
    float kr[HD], vr[HD];
    for (int kvh = 0; kvh < Hkv; kvh++) {
        for (int j = 0; j < S; j++) {
            const size_t row = size_t(kvh) * ldS + j;
            load_row(kc, kv_kind, dtype, row, kr);
            bool vloaded = false;
            float best = 0.0f;
            for (int g = 0; g < G; g++) {
                const int h = kvh * G + g;
                float t = canon_dot(&qn[size_t(h) * HD], kr);
                if (kv_kind == 0) t *= ks[row];
                if (g == 0 || t > best) best = t;
                const float a = std::max(t * scale, 0.0f), w = a * a;
                if (w != 0.0f) {
                    if (!vloaded) { load_row(vc, kv_kind, dtype, row, vr); vloaded = true; }
                    psum[h] += w;
                    const float wv = kv_kind == 0 ? w * vs[row] : w;
                    for (int d = 0; d < HD; d++) acc[size_t(h) * HD + d] += wv * vr[d];
                }
            }
            if (scores) scores[row] = best;
        }
    }
    for (int h = 0; h < Hq; h++) {
        const float den = std::sqrt(float(HD)) + psum[h];
        for (int d = 0; d < HD; d++) o[size_t(h) * HD + d] = store_act(acc[size_t(h) * HD + d] / den, dtype);
    }
}

// ---- key scoring on its own (sparse layers that hold their own 16-bit keys) --------------------
// The SCORES by-product of attn_full (attention.metal:189, 203-205) as a pass of its own:
// scores[kvh][j] = max over the kv head's query heads of q·k_j, ties keep the earlier head.
void orc_score_keys(const uint16_t* q, int dtype, int kv_kind, const void* kc, const float* ks,
                    int Hq, int Hkv, int S, int ldS, float* scores, int nthreads) {
    const int G = Hq / Hkv;
    std::vector<float> qn(size_t(Hq) * HD);
    for (int h = 0; h < Hq; h++) for (int d = 0; d < HD; d++) qn[size_t(h) * HD + d] = load_act(q[size_t(h) * HD + d], dtype);
    parallel_for(Hkv, nthreads, [&](int kvh) {
        float kr[HD];
        for (int j = 0; j < S; j++) {
            const size_t row = size_t(kvh) * ldS + j;
            load_row(kc, kv_kind, dtype, row, kr);
            float best = 0.0f;
            for (int g = 0; g < G; g++) {
                float t = canon_dot(&qn[size_t(kvh * G + g) * HD], kr);
                if (kv_kind == 0) t *= ks[row];
                if (g == 0 || t > best) best = t;
            }
            scores[row] = best;
        }
    });
}

// ---- key selection -----------------------------------------------------------------------------
// select_keys (attention.metal:680-744) per kv head over n = S - 128 scores: tau = the 1024-th
// largest order_bits among j < n; out = [j: bits_j > tau, ascending j] ++ [the first 1024 - count
// of j with bits_j == tau, ascending j] ++ [n, n+1, ..., n+127]. Requires S > 1152
// (Engine.swift:796). Written independently of the radix passes: an nth_element finds tau.
void orc_select_keys(const float* scores, int Hkv, int S, int ldS, uint32_t* idx) {
    const int n = S - RECENT;
    for (int kvh = 0; kvh < Hkv; kvh++) {
        const float* sc = scores + size_t(kvh) * ldS;
        uint32_t* out = idx + size_t(kvh) * (TOPK + RECENT);
        std::vector<uint32_t> bits(n);
        for (int j = 0; j < n; j++) bits[j] = order_bits(sc[j]);
        std::vector<uint32_t> tmp(bits);
        std::nth_element(tmp.begin(), tmp.begin() + (TOPK - 1), tmp.end(), std::greater<uint32_t>());
        const uint32_t tau = tmp[TOPK - 1];
        int g = 0;
        for (int j = 0; j < n; j++) if (bits[j] > tau) out[g++] = uint32_t(j);
        for (int j = 0; j < n && g < TOPK; j++) if (bits[j] == tau) out[g++] = uint32_t(j);
        for (int j = 0; j < RECENT; j++) out[TOPK + j] = uint32_t(n + j);
    }
}

// Engine.verifySelection (Engine.swift:1115-1131) as a property check. Returns 0 if the selection
// holds, else 1 + the failing rule (1 repeated rows, 2 recent rows, 3 a key below the top k, 4 count).
int orc_verify_selection(const float* scores, const uint32_t* idx, int Hkv, int S, int ldS) {
    const int k = TOPK, r = RECENT, n = S - r;
    if (S <= k + r) return -1;
    for (int h = 0; h < Hkv; h++) {
        const uint32_t* row = idx + size_t(h) * (k + r);
        std::vector<uint32_t> sorted(row, row + k + r);
        std::sort(sorted.begin(), sorted.end());
        if (std::adjacent_find(sorted.begin(), sorted.end()) != sorted.end()) return 1;
        for (int j = 0; j < r; j++) if (row[k + j] != uint32_t(n + j)) return 2;
        std::vector<float> s(scores + size_t(h) * ldS, scores + size_t(h) * ldS + n);
        std::vector<float> t(s);
        std::nth_element(t.begin(), t.begin() + (k - 1), t.end(), std::greater<float>());
        const float kth = t[k - 1];
        for (int j = 0; j < k; j++) if (row[j] >= uint32_t(n) || s[row[j]] < kth) return 3;
        int above = 0;
        for (int j = 0; j < n; j++) above += s[j] > kth;
        if (above > k) return 4;
    }
    return 0;
}

// ---- sparse layers, decode (softmax) -----------------------------------------------------------
// attn_sparse / attn_sparse8 / attn_sparse_short (attention.metal:370-441, 448-584, 593-645):
// rows = idx[kvh][0..nsel) when idx is given, else 0..S-1; s_r = q·k_r (· key scale) / sqrt(D);
// o = sum_r softmax(s)_r · v_r (· value scale), rounded to the storage dtype. The reference merges
// chunked online-softmax partials; the sum is the same, taken here with the exact maximum.
void orc_sparse_decode(const uint16_t* q, int dtype, int prenormed, const uint16_t* g1, const uint16_t* g2, int ng,
                       int kv_kind, const void* kc, const float* ks, const void* vc, const float* vs,
                       int Hq, int Hkv, int S, int ldS, const uint32_t* idx, int nsel, uint16_t* o) {
    const int G = Hq / Hkv;
    const float scale = 1.0f / std::sqrt(float(HD));
    const int R = idx ? nsel : S;
    std::vector<float> s(R);
    float qn[HD], kr[HD], vr[HD];
    for (int h = 0; h < Hq; h++) {
        const int kvh = h / G;
        prep_q(q + size_t(h) * HD, dtype, prenormed, g1, g2, ng, -1, qn);
        float M = NEG;
        for (int j = 0; j < R; j++) {
            const size_t row = size_t(kvh) * ldS + (idx ? idx[size_t(kvh) * nsel + j] : uint32_t(j));
            load_row(kc, kv_kind, dtype, row, kr);
            float t = canon_dot(qn, kr);
            if (kv_kind == 0) t *= ks[row];
            s[j] = t * scale;
            M = std::max(M, s[j]);
        }
        float L = 0.0f, acc[HD];
        for (int d = 0; d < HD; d++) acc[d] = 0.0f;
        for (int j = 0; j < R; j++) {
            const size_t row = size_t(kvh) * ldS + (idx ? idx[size_t(kvh) * nsel + j] : uint32_t(j));
            const float w = std::exp(s[j] - M);
            L += w;
            load_row(vc, kv_kind, dtype, row, vr);
            const float wv = kv_kind == 0 ? w * vs[row] : w;
            for (int d = 0; d < HD; d++) acc[d] += wv * vr[d];
        }
        for (int d = 0; d < HD; d++) o[size_t(h) * HD + d] = store_act(acc[d] / L, dtype);
    }
}

// ---- sliding layers ----------------------------------------------------------------------------
// The ring write of attn_sliding (attention.metal:47-62) / kv_sliding_b (prefill.metal:105-125)
// for T tokens at positions p0..: k = round(rope(norm(k)·(1+kg))), v as given, at slot pos % RING.
// `prenormed` stores k as given.
void orc_sliding_write(const uint16_t* k, const uint16_t* v, int ld_tok, int T, int dtype, int prenormed,
                       const uint16_t* kg, uint16_t* ring_k, uint16_t* ring_v, int p0, int RING, int Hkv) {
    for (int t = 0; t < T; t++) {
        const int pos = p0 + t, slot = pos % RING;
        for (int kvh = 0; kvh < Hkv; kvh++) {
            float kk[HD];
            const uint16_t* ksrc = k + size_t(t) * ld_tok + size_t(kvh) * HD;
            const uint16_t* vsrc = v + size_t(t) * ld_tok + size_t(kvh) * HD;
            for (int d = 0; d < HD; d++) kk[d] = load_act(ksrc[d], dtype);
            if (!prenormed) { head_norm(kk, kg, kg, 1, dtype); rope(kk, pos); }
            uint16_t* kd = ring_k + (size_t(kvh) * RING + slot) * HD;
            uint16_t* vd = ring_v + (size_t(kvh) * RING + slot) * HD;
            for (int d = 0; d < HD; d++) { kd[d] = store_act(kk[d], dtype); vd[d] = vsrc[d]; }
        }
    }
}

// Softmax attention of T tokens (positions p0..) over each one's last W positions, all already in
// the ring: attn_sliding's loop (attention.metal:63-101) and attn_sliding_b (prefill.metal:129-180).
// q is [T][ld_tok] with head h at h·128; o is [T][Hq·128].
void orc_sliding_attend(const uint16_t* q, int ld_tok, int T, int dtype, int prenormed, const uint16_t* qg,
                        const uint16_t* ring_k, const uint16_t* ring_v, int p0, int W, int RING,
                        int Hq, int Hkv, uint16_t* o, int nthreads) {
    const int G = Hq / Hkv;
    const float scale = 1.0f / std::sqrt(float(HD));
    parallel_for(T * Hq, nthreads, [&](int item) {
        const int t = item / Hq, h = item % Hq, kvh = h / G, pos = p0 + t;
        float qn[HD], kr[HD], vr[HD];
        prep_q(q + size_t(t) * ld_tok + size_t(h) * HD, dtype, prenormed, qg, qg, 1, pos, qn);
        const int n = std::min(pos + 1, W);
        std::vector<float> s(n);
        float M = NEG;
        for (int i = 0; i < n; i++) {
            const int slot = (pos - i) % RING;
            load_row(ring_k, 1, dtype, size_t(kvh) * RING + slot, kr);
            s[i] = canon_dot(qn, kr) * scale;
            M = std::max(M, s[i]);
        }
        float L = 0.0f, acc[HD];
        for (int d = 0; d < HD; d++) acc[d] = 0.0f;
        for (int i = 0; i < n; i++) {
            const int slot = (pos - i) % RING;
            const float w = std::exp(s[i] - M);
            L += w;
            load_row(ring_v, 1, dtype, size_t(kvh) * RING + slot, vr);
            for (int d = 0; d < HD; d++) acc[d] += w * vr[d];
        }
        uint16_t* od = o + (size_t(t) * Hq + h) * HD;
        for (int d = 0; d < HD; d++) od[d] = store_act(acc[d] / L, dtype);
    });
}

// ---- full layers, prefill chunk (causal ReLU²) -------------------------------------------------
// attn_full_b (prefill.metal:218-282) / relu2_prefill_nax (attn_nax.metal:228-270, 350-363) with
// threshold 0 and sink sqrt(D) (Prefill.swift:396-397): query row r (absolute position p0 + r)
// sees keys c <= p0 + r; out[r][h·128 + d] token-major. Rows r0, r0 + rstep, ... are computed
// (the others are left untouched), so a full-size chunk can be checked on a subset. `o_f32` (optional) receives
// the unrounded fp32 results.
static void full_prefill_impl(const uint16_t* q, int ld_tok, int Tq, int dtype, int prenormed,
                              const uint16_t* g1, const uint16_t* g2,
                              int kv_kind, const void* kc, const float* ks, const void* vc, const float* vs,
                              int Hq, int Hkv, int p0, int ldS, uint16_t* o, int r0, int rstep, int nthreads, float* o_f32,
                              bool qk8) {
    const int G = Hq / Hkv;
    const float scale = 1.0f / std::sqrt(float(HD));
    std::vector<int> rows;
    for (int r = r0; r < Tq; r += rstep) rows.push_back(r);
    parallel_for(int(rows.size()) * Hq, nthreads, [&](int item) {
        const int r = rows[item / Hq], h = item % Hq, kvh = h / G, S = p0 + r + 1;
        float qn[HD], kr[HD], vr[HD], acc[HD];
        int8_t q8[HD];
        float qscale = 0.0f;
        if (qk8) {
            // q_prep_b's QK8 branch (prefill.metal:421-422): the head-normed row (not yet rounded) through write_row8
            // (common.metal:74-84): rounded to the activation dtype, a = max |x|, codes rint(x 127 / a), scale a / 127
            const uint16_t* qr = q + size_t(r) * ld_tok + size_t(h) * HD;
            for (int d = 0; d < HD; d++) qn[d] = load_act(qr[d], dtype);
            if (!prenormed) head_norm(qn, g1, g2, 2, dtype);
            float a = 0.0f;
            for (int d = 0; d < HD; d++) { qn[d] = round_act(qn[d], dtype); a = std::max(a, std::fabs(qn[d])); }
            const float inv = a > 0.0f ? 127.0f / a : 0.0f;
            for (int d = 0; d < HD; d++) q8[d] = int8_t(int(std::rint(qn[d] * inv)));
            qscale = a / 127.0f;
        } else {
            prep_q(q + size_t(r) * ld_tok + size_t(h) * HD, dtype, prenormed, g1, g2, 2, -1, qn);
        }
        for (int d = 0; d < HD; d++) acc[d] = 0.0f;
        float psum = 0.0f;
        for (int j = 0; j < S; j++) {
            const size_t row = size_t(kvh) * ldS + j;
            float t;
            if (qk8) {
                // int8 x int8 -> int32 (attn_nax.metal:188-204), then x the row's query scale, x the key's scale
                const int8_t* k8 = static_cast<const int8_t*>(kc) + row * HD;
                int si = 0;
                for (int d = 0; d < HD; d++) si += int(q8[d]) * int(k8[d]);
                t = float(si) * qscale * ks[row];
            } else {
                load_row(kc, kv_kind, dtype, row, kr);
                t = canon_dot(qn, kr);
                if (kv_kind == 0) t *= ks[row];
            }
            const float a = std::max(t * scale, 0.0f), w = a * a;
            if (w != 0.0f) {
                psum += w;
                load_row(vc, kv_kind, dtype, row, vr);
                const float wv = kv_kind == 0 ? w * vs[row] : w;
                for (int d = 0; d < HD; d++) acc[d] += wv * vr[d];
            }
        }
        const float den = std::sqrt(float(HD)) + psum;
        uint16_t* od = o + (size_t(r) * Hq + h) * HD;
        for (int d = 0; d < HD; d++) od[d] = store_act(acc[d] / den, dtype);
        // the same quotient before it is rounded to the storage dtype, for tolerance checks on 16-bit outputs
        if (o_f32) for (int d = 0; d < HD; d++) o_f32[(size_t(r) * Hq + h) * HD + d] = acc[d] / den;
    });
}

void orc_full_prefill(const uint16_t* q, int ld_tok, int Tq, int dtype, int prenormed,
                      const uint16_t* g1, const uint16_t* g2,
                      int kv_kind, const void* kc, const float* ks, const void* vc, const float* vs,
                      int Hq, int Hkv, int p0, int ldS, uint16_t* o, int r0, int rstep, int nthreads, float* o_f32) {
    full_prefill_impl(q, ld_tok, Tq, dtype, prenormed, g1, g2, kv_kind, kc, ks, vc, vs, Hq, Hkv, p0, ldS, o, r0, rstep, nthreads, o_f32,
                      false);
}

// The reference's measurement-only QK8 build of the same kernel (attn_nax.metal:14-22, 62, 124-204; EMBLA_ATT8,
// Prefill.swift:142-144): Q Kᵀ in int8 with the query rows quantised by q_prep_b; int8 cache only.
void orc_full_prefill_qk8(const uint16_t* q, int ld_tok, int Tq, int dtype, int prenormed,
                          const uint16_t* g1, const uint16_t* g2,
                          const void* kc, const float* ks, const void* vc, const float* vs,
                          int Hq, int Hkv, int p0, int ldS, uint16_t* o, int r0, int rstep, int nthreads, float* o_f32) {
    full_prefill_impl(q, ld_tok, Tq, dtype, prenormed, g1, g2, 0, kc, ks, vc, vs, Hq, Hkv, p0, ldS, o, r0, rstep, nthreads, o_f32, true);
}

// ---- batched drivers for the timed CPU baseline ------------------------------------------------
// B independent sequences of orc_full_decode over `nthreads` host threads (one sequence a task).
void orc_full_decode_batch(int B, int nthreads, const uint16_t* q, int dtype,
                           const int8_t* kc, const float* ks, const int8_t* vc, const float* vs,
                           int Hq, int Hkv, int S, int ldS, uint16_t* o) {
    parallel_for(B, nthreads, [&](int b) {
        const size_t kvo = size_t(b) * Hkv * ldS;
        orc_full_decode(q + size_t(b) * Hq * HD, dtype, 1, nullptr, nullptr, 0, 0,
                        kc + kvo * HD, ks + kvo, vc + kvo * HD, vs + kvo, Hq, Hkv, S, ldS,
                        o + size_t(b) * Hq * HD, nullptr);
    });
}

// ---- the producer of q, k, v: the 4-bit GEMV (gemv / GemvRows, gemv.metal:37-92, common.metal:105-152) ----------
// words [rows][d_in / 32][4] 32-bit parts (word c, part k, nibble n: column 32 c + 8 k + n), scales and biases bfloat16
// [rows][d_in / 64]; x [tokens][ldx] and y [tokens][ldy] in the storage dtype. y = sum over words c of
// scale[c / 2] * (sum nibble * x) + bias[c / 2] * (sum x). The reference sums across a simdgroup in an unspecified order;
// here one fp32 chain per output: columns ascending inside a word (fmaf), the word's term a * dq + b * xs (one product, one
// fmaf), words ascending (plain adds), rounded to the storage dtype at the end (EPI 0).
void orc_w4_gemv(const uint32_t* words, const uint16_t* scales, const uint16_t* biases, int rows, int d_in,
                 const uint16_t* x, int ldx, int tokens, int dtype, uint16_t* y, int ldy, int nthreads) {
    const int nw = d_in / 32;
    parallel_for(tokens, nthreads, [&](int t) {
        std::vector<float> xf(d_in), xs(nw);
        for (int c = 0; c < d_in; c++) xf[c] = load_act(x[size_t(t) * ldx + c], dtype);
        for (int c = 0; c < nw; c++) {
            float s = 0.0f;
            for (int e = 0; e < 32; e++) s = s + xf[32 * c + e];
            xs[c] = s;
        }
        for (int r = 0; r < rows; r++) {
            float acc = 0.0f;
            for (int c = 0; c < nw; c++) {
                const uint32_t* w = words + (size_t(r) * nw + c) * 4;
                float dq = 0.0f;
                for (int k = 0; k < 4; k++)
                    for (int n = 0; n < 8; n++) dq = std::fmaf(float((w[k] >> (4 * n)) & 15u), xf[32 * c + 8 * k + n], dq);
                const float a = bf16_to_f(scales[size_t(r) * (nw / 2) + c / 2]), b = bf16_to_f(biases[size_t(r) * (nw / 2) + c / 2]);
                const float prod = a * dq;
                acc = acc + std::fmaf(b, xs[c], prod);
            }
            y[size_t(t) * ldy + r] = store_act(acc, dtype);
        }
    });
}

}  // extern "C"
