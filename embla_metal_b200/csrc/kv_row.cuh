// One key or value row of a new token, as one warp prepares it for the cache: a lane holds dims lane + 32 i like the
// reference's kernels (attention.metal:113-140, common.metal:30-41, 74-84). Every fp32 operation is an explicit
// round-to-nearest intrinsic in the order the CPU restatement uses, so rounded rows, codes and scales are bit-exact.
#pragma once

#include "common.cuh"

namespace embla {

// Loads the row; `norm`: head_norm without gains (keys), lane sums first, then the 32 lanes in lane order.
template <int DT>
__device__ __forceinline__ void kv_row_load(const void* src, size_t off, bool norm, int lane, float (&x)[4]) {
#pragma unroll
    for (int i = 0; i < 4; i++) x[i] = Act<DT>::load(src, off + lane + 32 * i);
    if (norm) {
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; i++) ss = __fadd_rn(ss, __fmul_rn(x[i], x[i]));
        float tot = 0.0f;
        for (int l = 0; l < 32; l++) tot = __fadd_rn(tot, __shfl_sync(0xffffffffu, ss, l));
        const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, float(HD)), EPS32)));
#pragma unroll
        for (int i = 0; i < 4; i++) x[i] = __fmul_rn(x[i], r);
    }
}

// write_row8 (common.metal:74-84): the row rounded to the activation dtype, a = max |x|, codes rint(x * 127 / a)
// (round half to even), scale a / 127; a zero row gives codes 0 and scale 0.
template <int DT>
__device__ __forceinline__ void kv_row_quantise(float (&x)[4], int (&code)[4], float& scale) {
    float a = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        x[i] = Act<DT>::round(x[i]);
        a = fmaxf(a, fabsf(x[i]));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
    const float inv = a > 0.0f ? __fdiv_rn(127.0f, a) : 0.0f;
#pragma unroll
    for (int i = 0; i < 4; i++) code[i] = int(rintf(__fmul_rn(x[i], inv)));
    scale = __fdiv_rn(a, 127.0f);
}

}  // namespace embla
