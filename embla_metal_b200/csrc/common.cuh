// Shared device/host helpers of the embla CUDA attention library (sm_100a only).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "embla_cuda_attn.h"

namespace embla {

constexpr int HD = EMBLA_HEAD_DIM;       // head dim
constexpr int BLK = EMBLA_BLOCK;         // positions per KV block
constexpr int CODE_BYTES = BLK * HD;     // int8 codes of one page side (K or V): 16 KiB
constexpr float EPS32 = 1.1920929e-07f;  // head-norm epsilon (common.metal:9)
constexpr float NEG_BIG = -1e30f;        // "-inf" of the running maxima (common.metal:10)

// Device-side error word values (EmblaAttn::err_dev).
constexpr int ERR_WAIT_FULL = 1, ERR_WAIT_EMPTY = 2, ERR_WAIT_DRAIN = 3;
// Bounded waits: tries before a kernel gives up, records an error and leaves; and the default bound in SM clocks
// (about half a second: one try may itself suspend the thread for a while). The clock bound is a launch
// parameter (KernelCtl::wait_cycles, embla_attn_set_wait_limit).
constexpr uint32_t WAIT_LIMIT = 1u << 20;
constexpr long long WAIT_CYCLES = 1ll << 30;

// Device timestamps a launch records when the profiler is on (trace_first / trace_last below).
constexpr int TRACE_SLOTS = 8;

// What every launch takes from its context besides its operands.
struct KernelCtl {
    int* err;                    // device error word
    unsigned long long* trace;   // TRACE_SLOTS device timestamps of this launch (trace_* below), or nullptr
    long long wait_cycles;       // bound of every device-side wait
    int stall_at;                // diagnostic (embla_attn_inject_stall): the producer stops issuing at this item of
                                 // its range, so that the consumers' bounded wait runs out; -1: never
    int early;                   // the launch may fetch its cache rows before the kernel ahead of it in the stream
                                 // has finished (that kernel writes none of them; set by the step driver)
    int l2_pages;                // early launches of the key-scoring pass: pages a CTA asks the L2 to fetch beyond its
                                 // shared-memory stages while it waits for the kernel ahead of it (the HBM idles during that
                                 // kernel's tail). Measured at 8 sequences: 8 pages take 1.5 of the pass's 44.5 microseconds;
                                 // the same request in the full-layer kernel, and requests for a later kernel's pages issued
                                 // from the selection, slowed their kernels down and sped nothing up.
};

// ---- host-side error plumbing -------------------------------------------------------------------
void set_error(const char* fmt, ...);
#define EMBLA_FAIL(status, ...)       \
    do {                              \
        ::embla::set_error(__VA_ARGS__); \
        return (status);              \
    } while (0)
#define EMBLA_CUDA_TRY(expr)                                                                         \
    do {                                                                                             \
        cudaError_t e_ = (expr);                                                                     \
        if (e_ != cudaSuccess) {                                                                     \
            ::embla::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e_), __FILE__, __LINE__); \
            return e_ == cudaErrorMemoryAllocation ? EMBLA_OOM : EMBLA_CUDA;                         \
        }                                                                                            \
    } while (0)

// The context's scratch and a pool's pages live on one device: a call made with another device current would launch
// there, with addresses that mean nothing on it.
#define EMBLA_CHECK_DEVICE(fn, ctx_, pool_)                                                                      \
    do {                                                                                                         \
        int dev_ = -1;                                                                                           \
        EMBLA_CUDA_TRY(cudaGetDevice(&dev_));                                                                    \
        if (dev_ != (ctx_)->device)                                                                              \
            EMBLA_FAIL(EMBLA_BAD_ARG, "%s: the context lives on device %d, the current device is %d", fn, (ctx_)->device, dev_); \
        if ((pool_) != nullptr && (pool_)->device != dev_)                                                       \
            EMBLA_FAIL(EMBLA_BAD_ARG, "%s: the pool lives on device %d, the current device is %d", fn, (pool_)->device, dev_);   \
    } while (0)

}  // namespace embla

// ---- handles --------------------------------------------------------------------------------------
struct EmblaKVPool {
    int n_layers, n_kv_heads, kv_dtype, scale_dtype, num_blocks;
    int scale_bytes;        // 2 or 4
    int rows_per_page;      // page bytes / 128
    size_t page_bytes, block_bytes, total_bytes;
    uint8_t* base;          // device
    CUtensorMap tmap_codes; // [total rows][128 B] uint8, box 256 rows, 128-byte swizzle
    CUtensorMap tmap_half;  // the same rows through a 128-row box (one side, K or V, of an int8 page)
    int device;
};

struct EmblaAttn {
    EmblaAttnConfig cfg;
    int device, sm_count;
    float* partials;        // split-K partial sums
    size_t partial_floats;
    int* counters;          // one arrival counter per (sequence, kv head); zero between launches
    int* err_dev;           // device error word
    int partial_slots;      // (sequence, kv head, key range) partials the scratch holds
    uint8_t* prefill_scratch;      // split-KV partials of the prefill kernel (embla_attn_reserve_prefill), then its arrival counters
    size_t prefill_scratch_bytes;  // bytes of the partials
    int prefill_counters;          // arrival counters behind them
    int pdl;                       // launches may start before the preceding kernel of the stream has drained (set by the step driver)
    int early;                     // the next launch may read its cache ahead of the kernel before it (set by the step driver per launch)
    long long wait_cycles;         // bound of the device-side waits of this context's launches
    int stall_at;                  // diagnostic stall of the next launches' producers (-1: off)
    int l2_pages;                  // pages an early key-scoring CTA asks the L2 for (EMBLA_L2_PAGES in the environment, default 8)
    // device-timestamp profiler (embla_attn_trace_*): 4 timestamps a launch, the entry point of each launch
    unsigned long long* trace_dev;
    int* trace_entry;              // host
    int trace_cap, trace_next, trace_on, trace_tag;
    // tensor maps of the sliding layers' rings seen so far (encoding two of them costs a few microseconds of host time a launch)
    struct RingMaps {
        const void* k;
        const void* v;
        long long seq_stride;
        int ring, n_kv_heads, batch;
        CUtensorMap mk, mv;
    };
    enum { RING_MAP_SLOTS = 32 };
    RingMaps ring_maps[RING_MAP_SLOTS];
    int ring_maps_used, ring_maps_next;
};

namespace embla {
// The control block of the context's next launch; takes the launch's trace slot when the profiler is on.
inline KernelCtl kernel_ctl(EmblaAttn* ctx) {
    KernelCtl c;
    c.err = ctx->err_dev;
    c.trace = nullptr;
    if (ctx->trace_on && ctx->trace_next < ctx->trace_cap) {
        ctx->trace_entry[ctx->trace_next] = ctx->trace_tag;
        c.trace = ctx->trace_dev + TRACE_SLOTS * size_t(ctx->trace_next++);
    }
    c.wait_cycles = ctx->wait_cycles;
    c.stall_at = ctx->stall_at;
    c.early = ctx->pdl ? ctx->early : 0;
    c.l2_pages = ctx->l2_pages;
    return c;
}
}  // namespace embla

namespace embla {

#ifdef __CUDACC__
// ---- activations --------------------------------------------------------------------------------
template <int DT> struct Act;
template <> struct Act<EMBLA_BF16> {
    __device__ static float load(const void* p, size_t i) { return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]); }
    __device__ static void store(void* p, size_t i, float v) { static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v); }
    __device__ static float round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
};
template <> struct Act<EMBLA_F16> {
    __device__ static float load(const void* p, size_t i) { return __half2float(static_cast<const __half*>(p)[i]); }
    __device__ static void store(void* p, size_t i, float v) { static_cast<__half*>(p)[i] = __float2half_rn(v); }
    __device__ static float round(float v) { return __half2float(__float2half_rn(v)); }
};

__device__ __forceinline__ float load_scale(const void* p, int i, int scale_bytes) {
    return scale_bytes == 4 ? static_cast<const float*>(p)[i] : __half2float(static_cast<const __half*>(p)[i]);
}

// ---- warp-level tensor-core tile: D[16x8] += A[16x16] * B[16x8], fp16 in, fp32 accumulate --------
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Two int8 codes -> half2, exactly: the bytes (offset to unsigned by ^0x80 beforehand) become the
// low mantissa bits of 1024.0, and 1152 = 1024 + 128 is subtracted.
constexpr uint32_t H2_1024 = 0x64646464u;   // byte source for the 0x64 exponent bytes
constexpr uint32_t H2_1152 = 0x64806480u;   // half2(1152, 1152)
__device__ __forceinline__ uint32_t h2_from_biased_bytes(uint32_t x, uint32_t sel) {
    uint32_t r = __byte_perm(x, H2_1024, sel), m = H2_1152;
    __half2 h = __hsub2(*reinterpret_cast<__half2*>(&r), *reinterpret_cast<__half2*>(&m));
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

// ---- shared-memory barriers and bulk (TMA) copies, every wait bounded ----------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
// (a barrier that is to be set up again must be invalidated first)
__device__ __forceinline__ void mbar_inval(uint64_t* bar) {
    asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Waits for the barrier's phase `parity`; gives up after WAIT_LIMIT tries or `limit` clocks, whichever comes first,
// and returns false.
__device__ __forceinline__ bool mbar_wait_bounded(long long limit, uint64_t* bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t i = 0; i < WAIT_LIMIT; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if (clock64() - t0 > limit) return false;
    }
    return false;
}

// ---- thread-block clusters: the hardware barrier over all CTAs of a cluster (threads that have exited do not count) and
// loads from another CTA's shared memory. No spinning: the barrier is a hardware wait like bar.sync.
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// the address, in the cluster's shared-memory window, of this CTA's shared address `saddr` in CTA `rank`
__device__ __forceinline__ uint32_t cluster_map(uint32_t saddr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}
__device__ __forceinline__ float cluster_ld_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void cluster_st_f32(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void cluster_st_u32(uint32_t addr, uint32_t v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
// adds into another CTA's shared memory without waiting for an answer
__device__ __forceinline__ void cluster_red_add_u32(uint32_t addr, uint32_t v) {
    asm volatile("red.shared::cluster.add.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}

// Partial sums that other CTAs left in global memory -> shared memory, every load of a batch in flight together (the
// last CTA of a split reads a few tens of KB once; read one dependent load at a time, that costs several microseconds).
template <int THREADS>
__device__ __forceinline__ void stage_from_global(float4* dst, const float4* src, int n4, int tid) {
    constexpr int BATCH = 12;
    for (int base = 0; base < n4; base += THREADS * BATCH) {
        float4 v[BATCH];
#pragma unroll
        for (int k = 0; k < BATCH; k++) {
            const int i = base + tid + THREADS * k;
            if (i < n4) v[k] = __ldcg(src + i);
        }
#pragma unroll
        for (int k = 0; k < BATCH; k++) {
            const int i = base + tid + THREADS * k;
            if (i < n4) dst[i] = v[k];
        }
    }
}

// ---- device-timestamp profiler: per launch, when the first CTA entered (0), when the first CTA was past its
// dependency wait (1), when the last CTA left its main loop (2) and when the last CTA finished (3), in nanoseconds of
// the GPU's global timer; slots 4-5 (first CTA to get there) and 6-7 (last CTA) are a kernel's own phase marks. The
// "last" slots hold the complement, so that one atomicMin serves all; the host presets every slot to all ones. Thread 0 of every CTA stamps; a launch without a slot (the usual case) pays one
// predictable branch.
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void trace_first(unsigned long long* tr, int slot) {
    if (tr != nullptr && threadIdx.x == 0) atomicMin(tr + slot, global_ns());
}
__device__ __forceinline__ void trace_last(unsigned long long* tr, int slot) {
    if (tr != nullptr && threadIdx.x == 0) atomicMin(tr + slot, ~global_ns());
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// 2-D tiled TMA load (no multicast): box at (x, y) of `map` into `dst`, completion on `bar`.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
// Programmatic dependent launch: a kernel launched with the stream-serialization attribute may become resident while the
// kernel before it in the stream drains. Every kernel of the decode step calls pdl_wait() before its first access to
// global memory (it returns once the preceding grid has completed and its writes are visible), then lets its own
// successor be scheduled. Both are no-ops in a launch without the attribute.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// 3-D tiled TMA load (no multicast): box at (x, y, z).
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
        : "memory");
}
// Asks the L2 to fetch `bytes` (a multiple of 16) at `src` (16-byte aligned) from memory; nothing waits for it.
__device__ __forceinline__ void l2_prefetch(const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(reinterpret_cast<uint64_t>(src)), "r"(bytes) : "memory");
}
// 1-D bulk copy global -> shared (both 16-byte aligned, bytes a multiple of 16).
__device__ __forceinline__ void bulk_load_1d(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
#endif  // __CUDACC__

// Host: a kernel launch, with the programmatic-dependent-launch attribute when `pdl`, as thread-block clusters of
// `cluster_x` CTAs along x when that is above 1.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel_cluster(bool pdl, int cluster_x, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                         cudaStream_t s, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute at[2];
    int n = 0;
    if (pdl) {
        at[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[n].val.programmaticStreamSerializationAllowed = 1;
        n++;
    }
    if (cluster_x > 1) {
        at[n].id = cudaLaunchAttributeClusterDimension;
        at[n].val.clusterDim.x = unsigned(cluster_x);
        at[n].val.clusterDim.y = 1;
        at[n].val.clusterDim.z = 1;
        n++;
    }
    cfg.attrs = at;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(bool pdl, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args&&... args) {
    return launch_kernel_cluster(pdl, 1, kern, grid, block, smem, s, static_cast<Args&&>(args)...);
}

// Host: the driver's cuTensorMapEncodeTiled, fetched through the runtime (no link against libcuda).
typedef CUresult (*TensorMapEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                           const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                           CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                           CUtensorMapFloatOOBfill);
TensorMapEncodeTiledFn tensor_map_encoder();

// full-layer (ReLU²) decode over a 16-bit pool (attn16_decode.cu), reached from embla_attn_full_decode
EmblaStatus attn16_full_decode(EmblaAttn* ctx, const EmblaKVPool* pool, const EmblaKVView* view, const EmblaQuery* q, void* o_dev,
                               int64_t o_stride, int max_len, cudaStream_t stream);

}  // namespace embla
