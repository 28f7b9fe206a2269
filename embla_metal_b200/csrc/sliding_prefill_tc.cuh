// Interface of the tcgen05 prefill kernel of the sliding layers (sliding_prefill_tc.cu) for its caller in
// sliding_prefill.cu.
#pragma once

#include "common.cuh"

namespace embla {

struct SlidingTcParams {
    const int32_t* pos0;
    const void* q;
    const void* g1;
    void* o;
    KernelCtl ctl;
    int64_t q_token_stride, q_seq_stride, o_token_stride, o_seq_stride;
    int n_tokens, n_kv_heads, G, prenormed, ring, window;
    float rope_freq[32];
};

// Launch for the whole batch on stream `s`.
EmblaStatus launch_sliding_prefill_tc(EmblaAttn* ctx, const EmblaRing* ring, const SlidingTcParams& p, int batch, cudaStream_t s);

}  // namespace embla
