// Helpers shared by the 16-bit-KV attention kernels (decode over gathered rows / rings, sliding prefill).
#pragma once

#include <cmath>

#include "common.cuh"

namespace embla {

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const uint32_t bytes = valid ? 16u : 0u;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}

__device__ __forceinline__ int rho16(int g) {   // as rho() of the full-layer kernel
    const int h = g >> 1, base = h < 2 ? 2 * h : 2 * h + 1;
    return base ^ ((g & 1) << 2);
}
__device__ __forceinline__ uint32_t movmatrix_trans16(uint32_t x) {
    uint32_t r;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(x));
    return r;
}

__device__ __forceinline__ uint32_t word4(const uint4& v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

template <int DT>
__device__ __forceinline__ void mma16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                      uint32_t b1) {
    if (DT == EMBLA_F16) {
        mma_16816(d, a0, a1, a2, a3, b0, b1);
    } else {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
}

template <int DT>
__device__ __forceinline__ uint32_t pack_act2(float lo, float hi) {
    if (DT == EMBLA_F16) return pack_h2(lo, hi);
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

// The query of one head in the reference's arithmetic: RMS norm with gains, optional RoPE at `pos`
// (pos < 0: none), rounded to the activation dtype. A lane holds dims lane + 32 i.
template <int DT>
__device__ __forceinline__ void norm_rope_round(float (&x)[4], const void* g1, const void* g2, int ng, int pos,
                                                const float* rope_freq, int lane) {
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; i++) ss = __fadd_rn(ss, __fmul_rn(x[i], x[i]));
    float tot = 0.0f;
    for (int l = 0; l < 32; l++) tot = __fadd_rn(tot, __shfl_sync(0xffffffffu, ss, l));
    const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, float(HD)), EPS32)));
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int d = lane + 32 * i;
        float gn = r;
        if (ng >= 1) gn = __fmul_rn(gn, __fadd_rn(1.0f, Act<DT>::load(g1, d)));
        if (ng >= 2) gn = __fmul_rn(gn, __fadd_rn(1.0f, Act<DT>::load(g2, d)));
        x[i] = __fmul_rn(x[i], gn);
    }
    if (pos >= 0) {   // common.metal:45-51: dims lane and lane + 32 rotate by -pos * freq[lane]
        const float theta = __fmul_rn(-float(pos), rope_freq[lane]);
        float sn, cs;
        sincosf(theta, &sn, &cs);
        const float x1 = x[0], x2 = x[1];
        x[0] = __fsub_rn(__fmul_rn(x1, cs), __fmul_rn(x2, sn));
        x[1] = __fadd_rn(__fmul_rn(x1, sn), __fmul_rn(x2, cs));
    }
#pragma unroll
    for (int i = 0; i < 4; i++) x[i] = Act<DT>::round(x[i]);
}

inline void fill_rope_freq(float* f) {
    // the reference's theta = -pos * exp2(-lane / 32 * log2(10000)) (common.metal:46), the factor in fp32
    for (int l = 0; l < 32; l++) f[l] = std::exp2(-float(l) / 32.0f * 13.287712379549449f);
}


}  // namespace embla
