/*
 * embla_cuda_attn.h — C ABI of the B200 (sm_100a) attention hot path for the embla engine.
 *
 * The reference engine (sevren-ai/embla-metal) has no plugin or FFI interface for attention: the
 * path sits behind two private Swift methods, Engine.encodeAttention (Sources/EmblaMetal/
 * Engine.swift:743-832) and Prefill.encode / encodeFullNAX (Sources/EmblaMetal/Prefill.swift:265-407),
 * which bind buffers and dispatch Metal kernels. This header gives one entry point per kernel
 * dispatch of those methods, with the same operands, so that a Swift caller can replace each
 * `dispatchThreadgroups` with one C call through a module map and a thin Swift wrapper.
 *
 * Conventions
 *  - Every function returns an EmblaStatus (0 = ok) and never aborts or throws; a message for the
 *    last failure of the calling thread is available from embla_last_error(). (The reference
 *    throws at init, MetalContext.swift:78-90, and traps on a failed command buffer,
 *    Engine.swift:1070, 1170.)
 *  - All pointers named *_dev are device pointers owned by the caller unless stated otherwise.
 *    Work is enqueued on the given CUDA stream (a cudaStream_t passed as void*) and the call
 *    returns without synchronising, like encoding into a Metal command buffer.
 *  - A handle is not thread-safe; distinct handles may be used from distinct threads/streams.
 *  - Activations are 16-bit (bfloat16 as in the reference, or float16); head_dim is 128.
 *  - Batched: every call takes `batch` independent sequences (the reference runs one).
 *    `seq_lens_dev[b]` is the number of keys the call sees for sequence b, the current token
 *    included — the reference's AttnParams.S = pos + 1 (Engine.swift:796-801).
 *
 * KV cache layout (replaces Engine.swift:269-284 and the span lists of PrefixCache.swift:153-186)
 *  - A pool holds `num_blocks` physical blocks. A block covers 128 consecutive positions of one
 *    sequence for every layer of the pool and every kv head, and is contiguous in memory:
 *        block = [layer][kv head] pages;  int8 page = K codes [128][128] | V codes [128][128] |
 *        K scales [128] | V scales [128]   (scales fp32 as the reference, or fp16).
 *    A sequence is a row of a block table (int32 physical block ids, position p lives in entry
 *    p / 128). A prefix-cache hit is a block-table edit (share) or one contiguous copy
 *    (embla_kv_block_export / _import), where the reference blits ~40 spans per block.
 */
#ifndef EMBLA_CUDA_ATTN_H
#define EMBLA_CUDA_ATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    EMBLA_OK = 0,
    EMBLA_BAD_ARG = 1,
    EMBLA_OOM = 2,
    EMBLA_CUDA = 3,      /* a CUDA runtime / driver call failed */
    EMBLA_NCCL = 4,
    EMBLA_TIMEOUT = 5,   /* a bounded device-side wait ran out (see embla_attn_check) */
    EMBLA_UNSUPPORTED = 6
} EmblaStatus;

enum { EMBLA_BF16 = 0, EMBLA_F16 = 1 };                       /* activation dtype */
enum { EMBLA_KV_INT8 = 0, EMBLA_KV_16BIT = 1 };               /* cache element type (16BIT = activation dtype) */
enum { EMBLA_SCALE_F32 = 0, EMBLA_SCALE_F16 = 1 };            /* int8 row scale dtype */
enum { EMBLA_HEAD_DIM = 128, EMBLA_BLOCK = 128, EMBLA_TOPK = 1024, EMBLA_RECENT = 128 };
/* Longest sequence embla_select_keys ranks: a (sequence, kv head) pair's keys are held in the registers of a
 * cluster of at most 8 CTAs x 1024 threads x 32 keys, plus the 128 latest. (The reference's loop takes any
 * length, attention.metal:701; its engine is built for 32768.) */
enum { EMBLA_SELECT_MAX_KEYS = 8 * 1024 * 32 + 128 };

typedef struct EmblaAttn EmblaAttn;       /* context: device, scratch (split-K partials, counters) */
typedef struct EmblaKVPool EmblaKVPool;   /* paged KV pool */

/* Model shape of the path; the counterpart of `enum Embla` (Engine.swift:7-27) for attention. */
typedef struct {
    int32_t n_q_heads;     /* 16 */
    int32_t n_kv_heads;    /* 4 (the reference's full/sparse layers use 2) */
    int32_t act_dtype;     /* EMBLA_BF16 | EMBLA_F16 */
    int32_t max_batch;     /* sequences per call; sizes the scratch */
    int32_t max_context;   /* keys per sequence; sizes the scratch */
} EmblaAttnConfig;

/* Queries of a call. `prenormed` = 0 reproduces the reference: the kernel applies the per-head RMS
 * norm with gains (1 + g1)(1 + g2) (`ng` of them; common.metal:30-41) and rounds to the activation
 * dtype before use (attention.metal:166-169). `prenormed` = 1 takes q as given. */
typedef struct {
    const void* q_dev;        /* [batch][q_stride] elements, head h at h * 128 (the reference's qkv buffer) */
    int64_t     q_stride;     /* elements between sequences (4096 for the reference's qkv rows) */
    int32_t     prenormed;
    int32_t     ng;           /* 0, 1 or 2 gain vectors */
    const void* g1_dev;       /* [128] gains, activation dtype; may be NULL when ng < 1 */
    const void* g2_dev;       /* [128]; may be NULL when ng < 2 */
} EmblaQuery;

/* A sequence batch's view of a pool: which blocks, how many keys. */
typedef struct {
    const int32_t* block_table_dev;   /* [batch][table_stride] physical block ids */
    int32_t        table_stride;
    const int32_t* seq_lens_dev;      /* [batch] keys visible (current token included) */
    int32_t        batch;
    int32_t        layer;             /* layer index inside the pool */
    int32_t        max_seq_len;       /* host-side upper bound of seq_lens (sizes the key split);
                                         0 = the context's max_context */
} EmblaKVView;

/* ---- lifetime ---------------------------------------------------------------------------------- */
const char* embla_version(void);
/* Message of the calling thread's last failing call (never NULL). */
const char* embla_last_error(void);

/* Replaces Engine.init's pipeline + scratch set-up for attention (Engine.swift:221-230, 242-258:
 * `apart`, `counter`, `scores`, `sel`). Allocates split-K scratch on the current device. */
EmblaStatus embla_attn_create(const EmblaAttnConfig* cfg, EmblaAttn** out);
void        embla_attn_destroy(EmblaAttn* ctx);
/* Reads (and clears) the device-side error word: EMBLA_TIMEOUT if a bounded wait of an earlier
 * kernel ran out. Synchronises the stream. */
EmblaStatus embla_attn_check(EmblaAttn* ctx, void* stream);
/* Every device-side wait of this library's kernels (on a shared-memory barrier that a TMA copy or
 * another warp completes) is bounded; a wait that runs out makes the kernel record an error code, wait
 * (bounded again) for its own copies in flight and return, and embla_attn_check reports EMBLA_TIMEOUT.
 * `cycles` is that bound in SM clocks for the launches this context makes from now on (default 2^30,
 * about half a second). The counterpart of the reference's trap on a failed command buffer
 * (Engine.swift:1070, 1170), without losing the context. */
EmblaStatus embla_attn_set_wait_limit(EmblaAttn* ctx, int64_t cycles);
/* Diagnostic, for testing the path above without any fault: the producer warps of the launches this
 * context makes from now on stop requesting data at item `item` of their range (page of a key range,
 * tile of a window), so that the consumers' wait for it runs out. -1 turns it off.
 * EMBLA_STALL_PARTIALS (an item no producer reaches) instead keeps the page ranges of a prefill unit that
 * meet in the scratch from reporting their partial sums, so that the wait of the unit's last range, the
 * only wait of one CTA for others in this library, runs out. */
#define EMBLA_STALL_PARTIALS (1 << 30)
EmblaStatus embla_attn_inject_stall(EmblaAttn* ctx, int32_t item);

/* Device-timestamp profiler, the counterpart of the reference's per-part Profiler (StepEncoder.swift:7-65)
 * that does not serialise the launches it measures: between trace_begin and trace_end every launch
 * of this context (at most max_launches of them) records times of the GPU's global nanosecond timer:
 * [0] the first CTA entering, [1] the first CTA past its wait for the preceding kernel, [2] the last CTA
 * leaving its main loop, [3] the last CTA finishing, [4..7] a kernel's own phase marks (4, 5: first CTA
 * to get there; 6, 7: last; 0 where a kernel has none). trace_begin allocates on first use or growth
 * (it then synchronises the stream); trace_end synchronises the stream and writes
 * stamps[launch][EMBLA_TRACE_SLOTS] and the entry point of each launch (EMBLA_ENTRY_* inside
 * embla_stack_decode_step, else -1). */
enum { EMBLA_TRACE_SLOTS = 8 };
EmblaStatus embla_attn_trace_begin(EmblaAttn* ctx, int32_t max_launches, void* stream);
EmblaStatus embla_attn_trace_end(EmblaAttn* ctx, void* stream, uint64_t* stamps, int32_t* entries, int32_t cap,
                                 int32_t* n_launches);

/* Replaces the cache allocation of Engine.swift:269-284 for the full layers. */
EmblaStatus embla_kv_pool_create(int32_t n_layers, int32_t n_kv_heads, int32_t kv_dtype, int32_t scale_dtype,
                                 int32_t num_blocks, EmblaKVPool** out);
void        embla_kv_pool_destroy(EmblaKVPool* pool);
/* Bytes of one physical block, and of one (layer, kv head) page inside it. */
size_t      embla_kv_block_bytes(const EmblaKVPool* pool);
size_t      embla_kv_page_bytes(const EmblaKVPool* pool);
/* Device address of the pool (block 0), for tests and for callers that fill pages themselves. */
void*       embla_kv_pool_base(const EmblaKVPool* pool);

/* Replaces Engine.copy over fullSpans (PrefixCache.swift:153-168, 200-212): one block out of / into
 * the pool as one contiguous copy. `dst`/`src` may be host (pinned or pageable) or device memory. */
EmblaStatus embla_kv_block_export(const EmblaKVPool* pool, int32_t block, void* dst, void* stream);
EmblaStatus embla_kv_block_import(EmblaKVPool* pool, int32_t block, const void* src, void* stream);

/* ---- KV append ---------------------------------------------------------------------------------- */
/* Replaces kv_append (attention.metal:113-140) and kv_append_b (prefill.metal:184-212) with
 * write_row8 (common.metal:74-84): for each sequence b and token t < n_tokens at position
 * pos0_dev[b] + t, quantises the k and v rows of every kv head into the view's layer.
 * `norm_k` = 1 RMS-norms k without gains first, as the reference does. k/v are
 * [batch][n_tokens][stride] elements with kv head h at h * 128. Codes and scales are bit-exact
 * against the reference arithmetic. seq_lens_dev of the view is not read. */
EmblaStatus embla_kv_append(EmblaAttn* ctx, EmblaKVPool* pool, const EmblaKVView* view,
                            const int32_t* pos0_dev, int32_t n_tokens,
                            const void* k_dev, const void* v_dev, int64_t token_stride, int64_t seq_stride,
                            int32_t norm_k, void* stream);

/* ---- the producer of q, k, v: 4-bit stacked GEMV ---------------------------------------------------- */
/* One 4-bit matrix of the model as the reference stores it (GemvRows, common.metal:105-152; Seg, gemv.metal:21-27):
 * `rows` rows of d_in four-bit values in d_in / 32 words of 16 bytes (word c, 32-bit part k, nibble n: column
 * 32 c + 8 k + n), with one bfloat16 scale and one bfloat16 bias per row and 64 columns:
 * y[row] = sum over words c of scale[c / 2] * (sum nibble * x) + bias[c / 2] * (sum x). */
typedef struct {
    const void* words_dev;    /* [rows][d_in / 32] x 16 bytes, 16-byte aligned */
    const void* scales_dev;   /* bfloat16 [rows][d_in / 64] */
    const void* biases_dev;   /* bfloat16 [rows][d_in / 64] */
    int32_t     rows;         /* q: n_q_heads * 128; k, v: n_kv_heads * 128 */
} EmblaW4Matrix;
/* Replaces the stacked q/k/v dispatch of gemv (gemv.metal:37-92, EPI 0; Engine.swift:746-752) for `batch` tokens: x_dev
 * [batch][x_stride] in the activation dtype, outputs rounded to it into qkv_dev [batch][qkv_stride] (q heads, k heads,
 * v heads, 128 each). Every output is one fp32 chain in a fixed order, equal bit for bit to the CPU restatement. */
EmblaStatus embla_qkv_project(EmblaAttn* ctx, const EmblaW4Matrix* wq, const EmblaW4Matrix* wk, const EmblaW4Matrix* wv,
                              int32_t d_in, const void* x_dev, int64_t x_stride, int32_t batch, void* qkv_dev,
                              int64_t qkv_stride, void* stream);
/* The same for a full layer with the attention side's work on the rows folded into the GEMV's epilogue (no counterpart in
 * the reference, which runs kv_append and the in-kernel head norm after it): q is head-normed with `gains` (g1, g2; NULL or
 * prenormed: stored as computed) and stored as the prenormed queries of embla_attn_full_decode; k (normed first when
 * norm_k) and v of the token at position seq_lens_dev[b] - 1 are quantised and written into the view's layer of the int8
 * pool, the same bytes embla_kv_append writes from the rows embla_qkv_project stores; the k and v slots of qkv_dev are
 * left untouched. batch = view->batch. */
EmblaStatus embla_qkv_project_full_step(EmblaAttn* ctx, const EmblaW4Matrix* wq, const EmblaW4Matrix* wk,
                                        const EmblaW4Matrix* wv, int32_t d_in, const void* x_dev, int64_t x_stride,
                                        const EmblaQuery* gains, EmblaKVPool* pool, const EmblaKVView* view,
                                        int32_t norm_k, void* qkv_dev, int64_t qkv_stride, void* stream);

/* The same for a sliding layer (declared after EmblaRing below): embla_qkv_project_sliding_step. */
/* Replaces the o-projection after attention (gemv with EPI 3 or 2, gemv.metal:85-88; Engine.swift:830): the 4-bit GEMV of
 * the attention output rows o_dev [batch][o_stride] (activation dtype, d_in = n_q_heads * 128 values), each output rounded
 * to the activation dtype and stored into (accumulate = 0) or added to (1) the fp32 residual rows x_dev [batch][x_stride]. */
EmblaStatus embla_oproj(EmblaAttn* ctx, const EmblaW4Matrix* wo, int32_t d_in, const void* o_dev, int64_t o_stride,
                        int32_t batch, float* x_dev, int64_t x_stride, int32_t accumulate, void* stream);

/* ---- decode, full layers (ReLU²) ------------------------------------------------------------------ */
/* Replaces attn_full8 (attention.metal:235-363; dispatch Engine.swift:796-818): ReLU² attention
 * of one query token per sequence over the int8 cache, split over key ranges with a deterministic
 * combine. o_dev is [batch][o_stride] elements, head h at h * 128. When `scores_dev` is not NULL
 * (the reference's SCORES variant, attention.metal:146, 296-306) the kernel also writes
 * scores[b][kv head][j] = max over the kv head's query heads of q·k_j·kscale_j for j < seq_len,
 * rows of `scores_stride` floats, bit-exact against the oracle's summation order.
 * A 16-bit pool is served too: the reference's build without the int8 cache (EMBLA_KV8=0, Engine.swift:163: attn_full,
 * attention.metal:148-220), the rows in the activation dtype and no scales; the scores then come from a scoring pass of
 * their own ahead of the attention (queries prenormed), and embla_attn_full_step is refused (embla_kv_append first). */
EmblaStatus embla_attn_full_decode(EmblaAttn* ctx, const EmblaKVPool* pool, const EmblaKVView* view,
                                   const EmblaQuery* q, void* o_dev, int64_t o_stride,
                                   float* scores_dev, int64_t scores_stride, void* stream);

/* The reference's per-layer pair kv_append + attn_full8 (Engine.swift:756-762, 796-818) in one launch: the current
 * token of every sequence (position seq_lens_dev[b] - 1) is quantised from its raw k and v rows (k_dev, v_dev:
 * [batch][kv_stride] elements, kv head h at h * 128; `norm_k` as embla_kv_append) into the view's layer, and the
 * attention sees it. Same result as embla_kv_append followed by embla_attn_full_decode. */
EmblaStatus embla_attn_full_step(EmblaAttn* ctx, EmblaKVPool* pool, const EmblaKVView* view, const EmblaQuery* q,
                                 const void* k_dev, const void* v_dev, int64_t kv_stride, int32_t norm_k,
                                 void* o_dev, int64_t o_stride, float* scores_dev, int64_t scores_stride, void* stream);

/* No counterpart in the reference (its engine owns every buffer and allocates them all at init).
 * The same attention as embla_attn_full_decode (without scores) for callers that cannot allocate
 * device memory where they run attention — a server that gave all device memory to its own arena at
 * start-up, or a thread in which cudaMalloc and the synchronisation it may imply are forbidden. It
 * takes no context: the split-K partial sums and arrival counters live in a fixed array inside the
 * library (about 4.1 MiB, held by every GPU that loads the library until the process exits), and
 * the call makes no cudaMalloc / cudaFree or any other allocating call.
 *  - Limit: batch * n_kv_heads <= 256 (sequence, kv head) pairs; more is refused with EMBLA_BAD_ARG.
 *    view->max_seq_len must be given. The model shape comes from `n_q_heads` (kv heads from the pool)
 *    and `act_dtype`.
 *  - The first call on a device resolves the array's address and configures the kernels; make that
 *    call before any stream capture, and from one thread: two threads making a device's first call at
 *    the same moment race on that set-up.
 *  - All calls on a device share the array: two calls whose kernels may overlap on the GPU (different
 *    streams) race on it. Calls on one stream are safe; each call clears the counters first.
 *  - A bounded device-side wait that runs out is not reported by this variant (there is no context
 *    to ask); use embla_attn_full_decode + embla_attn_check where that matters. */
EmblaStatus embla_attn_full_decode_noalloc(const EmblaKVPool* pool, const EmblaKVView* view, const EmblaQuery* q,
                                           int32_t n_q_heads, int32_t act_dtype, void* o_dev, int64_t o_stride,
                                           void* stream);

/* ---- key scoring and selection (sparse layers) --------------------------------------------------- */
/* The SCORES by-product of attn_full (attention.metal:146, 189, 203-205) as a pass of its own, for
 * sparse layers that keep their own 16-bit keys in a EMBLA_KV_16BIT pool: scores[b][kv head][j] =
 * max over the kv head's query heads of q·k_j for j < seq_len. q is taken as given ([batch][q_stride],
 * head h at h * 128). Bit-exact against the oracle's summation order. */
EmblaStatus embla_score_keys(EmblaAttn* ctx, const EmblaKVPool* pool, const EmblaKVView* view,
                             const void* q_dev, int64_t q_stride, float* scores_dev, int64_t scores_stride,
                             void* stream);

/* embla_kv_append of the current token (position seq_lens_dev[b] - 1; raw rows k_dev, v_dev: [batch][kv_stride]
 * elements, kv head h at h * 128; `norm_k` as embla_kv_append) into the 16-bit pool and embla_score_keys in one launch;
 * the appended key is scored too, and the row is in the pool for the attention that follows. */
EmblaStatus embla_score_keys_step(EmblaAttn* ctx, EmblaKVPool* pool, const EmblaKVView* view, const void* q_dev,
                                  int64_t q_stride, const void* k_dev, const void* v_dev, int64_t kv_stride,
                                  int32_t norm_k, float* scores_dev, int64_t scores_stride, void* stream);

/* Replaces select_keys (attention.metal:655-744; dispatch Engine.swift:819-827): for every sequence
 * with seq_len > 1152 and every kv head, idx[b][kv head][0..1151] = the 1024 highest-scoring keys among
 * j < seq_len - 128 (ties: lowest index; order: greater ascending, then equal ascending), then the 128
 * latest. Rows of shorter sequences are left untouched (the reference does not select yet,
 * Engine.swift:796). scores rows are scores_stride floats apart per (sequence, kv head). Exact.
 * max_seq_len (or the context's max_context when 0) above EMBLA_SELECT_MAX_KEYS is refused with
 * EMBLA_UNSUPPORTED; embla_stack_create refuses such a context for a stack with selecting layers. */
EmblaStatus embla_select_keys(EmblaAttn* ctx, const float* scores_dev, int64_t scores_stride,
                              const int32_t* seq_lens_dev, int32_t batch, int32_t max_seq_len,
                              uint32_t* idx_dev, void* stream);

/* ---- decode, sparse layers (softmax) ---------------------------------------------------------------- */
/* Replaces attn_sparse / attn_sparse8 / attn_sparse_short (attention.metal:370-441, 448-584, 593-645;
 * dispatch Engine.swift:796-818) over a EMBLA_KV_16BIT pool: softmax attention over all keys of a
 * sequence with at most 1152, else over its selected rows idx[b][kv head][0..1151]. */
EmblaStatus embla_attn_sparse_decode(EmblaAttn* ctx, const EmblaKVPool* pool, const EmblaKVView* view,
                                     const EmblaQuery* q, const uint32_t* idx_dev, void* o_dev, int64_t o_stride,
                                     void* stream);

/* The same over the preceding full layer's int8 cache, as the reference's sparse layers run
 * (Engine.swift:461-462; attn_sparse8 / attn_sparse_short, attention.metal:448-584, 593-645): the rows come
 * from embla_select_keys applied to the scores embla_attn_full_decode wrote for that full layer. */
EmblaStatus embla_attn_sparse_decode_int8(EmblaAttn* ctx, const EmblaKVPool* pool, const EmblaKVView* view,
                                          const EmblaQuery* q, const uint32_t* idx_dev, void* o_dev, int64_t o_stride,
                                          void* stream);

/* ---- sliding layers ------------------------------------------------------------------------------------ */
/* The sliding layers' rings (Engine.swift:269-276; RING = 4096, attention.metal:4-6): per sequence
 * [n_kv_heads][ring][128] keys and the same for values, in the activation dtype, owned by the caller. */
typedef struct {
    void*   k_dev;
    void*   v_dev;
    int64_t seq_stride;   /* elements between sequences (>= n_kv_heads * ring * 128) */
    int32_t ring;         /* slots; must hold window + one prefill chunk */
    int32_t window;       /* positions attended, the current one included (128 in the reference) */
} EmblaRing;

/* Replaces the ring write of attn_sliding (attention.metal:47-62) and kv_sliding_b (prefill.metal:105-125):
 * for token t < n_tokens of sequence b at position pos0_dev[b] + t, k = round(rope(norm(k) (1 + kgain)))
 * and v go to slot pos % ring. `prenormed` stores k as given. k/v are [batch][n_tokens][stride]. */
EmblaStatus embla_sliding_write(EmblaAttn* ctx, const EmblaRing* ring, const int32_t* pos0_dev, int32_t batch,
                                int32_t n_tokens, const void* k_dev, const void* v_dev, int64_t token_stride,
                                int64_t seq_stride, int32_t prenormed, const void* kgain_dev, void* stream);

/* embla_qkv_project for a sliding layer with the ring write of attn_sliding (attention.metal:47-62) in its epilogue: q is
 * normed with qgain_dev, rotated at the token's position seq_lens_dev[b] - 1, rounded and stored as the prenormed query of
 * embla_attn_sliding_decode; k is normed with kgain_dev, rotated and rounded, v rounded, and both are written to the ring
 * slot of that position (NULL gains: the rows are stored as computed). The k and v slots of qkv_dev are left untouched. */
EmblaStatus embla_qkv_project_sliding_step(EmblaAttn* ctx, const EmblaW4Matrix* wq, const EmblaW4Matrix* wk,
                                           const EmblaW4Matrix* wv, int32_t d_in, const void* x_dev, int64_t x_stride,
                                           const void* qgain_dev, const void* kgain_dev, const EmblaRing* ring,
                                           const int32_t* seq_lens_dev, int32_t batch, void* qkv_dev, int64_t qkv_stride,
                                           void* stream);

/* Replaces the attention of attn_sliding (attention.metal:63-101): softmax over the last
 * min(seq_len, window) positions, which must already be in the ring (embla_sliding_write first).
 * Without `prenormed`, q is normed with gain g1, rotated at position seq_len - 1 and rounded. */
EmblaStatus embla_attn_sliding_decode(EmblaAttn* ctx, const EmblaRing* ring, const int32_t* seq_lens_dev,
                                      int32_t batch, const EmblaQuery* q, void* o_dev, int64_t o_stride,
                                      void* stream);

/* Replaces attn_sliding as the reference runs it (attention.metal:26-102; dispatch Engine.swift:771-780): the ring
 * write of the current token and the attention in ONE launch. k_dev / v_dev are the current token's raw rows
 * ([batch][kv_stride], kv head h at h * 128); the key is normed with kgain, rotated at position seq_len - 1 and rounded
 * (or stored as given with k_prenormed), written to slot (seq_len - 1) % ring, and used from registers by the attention. */
EmblaStatus embla_attn_sliding_step(EmblaAttn* ctx, const EmblaRing* ring, const int32_t* seq_lens_dev, int32_t batch,
                                    const EmblaQuery* q, const void* k_dev, const void* v_dev, int64_t kv_stride,
                                    int32_t k_prenormed, const void* kgain_dev, void* o_dev, int64_t o_stride,
                                    void* stream);

/* ---- prefill chunk, sliding layers ------------------------------------------------------------------- */
/* Replaces attn_sliding_b / attn_sliding8_b (prefill.metal:129-180, 439-548; dispatch Prefill.swift:300-313):
 * token t of sequence b, at position pos0_dev[b] + t, attends its last `window` positions with softmax. The
 * chunk's keys and values must already be in the ring (embla_sliding_write with n_tokens first, as the
 * reference runs kv_sliding_b first); the ring must hold window + n_tokens slots. Without `prenormed`, q is
 * normed with gain g1 (ng = 1), rotated at its position and rounded. Layout of q and o as for
 * embla_attn_full_prefill. */
EmblaStatus embla_attn_sliding_prefill(EmblaAttn* ctx, const EmblaRing* ring, const int32_t* pos0_dev, int32_t batch,
                                       int32_t n_tokens, const EmblaQuery* q, int64_t q_token_stride, void* o_dev,
                                       int64_t o_token_stride, int64_t o_seq_stride, void* stream);

/* ---- prefill chunk, full layers (causal ReLU²) -------------------------------------------------------- */
/* Replaces q_prep_b + relu2_prefill_nax (prefill.metal:408-426, attn_nax.metal:61-364; dispatch
 * Prefill.swift:378-407) and the fallback attn_full_b (prefill.metal:218-282): for each sequence, the
 * n_tokens new tokens at positions pos0_dev[b] + t attend causally (keys <= their own position) over the
 * int8 cache, which must already hold their own keys and values (embla_kv_append first, as the reference
 * runs kv_append_b first). Token t's query head h is at q_dev[b * q->q_stride + t * q_token_stride +
 * h * 128]; out is token-major, o_dev[b * o_seq_stride + t * o_token_stride + h * 128]. Strides are in
 * elements and must be multiples of 8. Runs on tcgen05 tensor cores with fp32 accumulation in TMEM. */
EmblaStatus embla_attn_full_prefill(EmblaAttn* ctx, const EmblaKVPool* pool, const EmblaKVView* view,
                                    const int32_t* pos0_dev, int32_t n_tokens, const EmblaQuery* q,
                                    int64_t q_token_stride, void* o_dev, int64_t o_token_stride,
                                    int64_t o_seq_stride, void* stream);
/* No counterpart in the reference (it runs one GPU): embla_attn_full_prefill for a chunk sharded over several GPUs by kv
 * head. Besides o_dev, every output row is stored, by the kernel's own epilogue and with plain stores over NVLink, to
 * o_peers_dev[i] for i < n_peers (at most 8; a host array of device addresses): each the address, in another GPU's memory
 * mapped into this process (CUDA IPC, symmetric memory, peer access), of the place of THIS rank's rows in that GPU's
 * token-major output, addressed with the same strides as o_dev. The compute and the all-gather of the per-head outputs are
 * then one kernel: when every rank's call has completed (a barrier across the GPUs after it, which is the caller's, as
 * is not overwriting a peer's output that the peer still reads), every GPU holds the whole o[T][n_q_heads * 128]. */
EmblaStatus embla_attn_full_prefill_scatter(EmblaAttn* ctx, const EmblaKVPool* pool, const EmblaKVView* view,
                                            const int32_t* pos0_dev, int32_t n_tokens, const EmblaQuery* q,
                                            int64_t q_token_stride, void* o_dev, void* const* o_peers_dev, int32_t n_peers,
                                            int64_t o_token_stride, int64_t o_seq_stride, void* stream);
/* The reference's int8 Q Kᵀ build of the same kernel (QK8: attn_nax.metal:14-22, 62, 124-204, with q_prep_b's QK8
 * branch, prefill.metal:421-422; switched on by EMBLA_ATT8, Prefill.swift:142-144; measurement-only there): every
 * query row is quantised like a cache row (rounded to the activation dtype, codes rint(x 127 / max|x|), scale
 * max|x| / 127), Q Kᵀ runs in int8 on the cache's codes as they are (tcgen05.mma kind::i8, int32 accumulators: the dots
 * are exact), and a score is dot x query scale x key scale / sqrt(128). P V as in embla_attn_full_prefill. Same
 * operands; the result differs from embla_attn_full_prefill's by the quantisation of the queries. */
EmblaStatus embla_attn_full_prefill_qk8(EmblaAttn* ctx, const EmblaKVPool* pool, const EmblaKVView* view,
                                        const int32_t* pos0_dev, int32_t n_tokens, const EmblaQuery* q,
                                        int64_t q_token_stride, void* o_dev, int64_t o_token_stride,
                                        int64_t o_seq_stride, void* stream);
/* Part of Engine.init's scratch set-up (`apart`, Engine.swift:242-258) that only prefill needs: about 39 MB of
 * partial sums, with which embla_attn_full_prefill cuts the pages of a (256 tokens, head) unit over several CTAs
 * when a chunk has fewer units than the GPU has SMs (short chunks, head-sharded prefill). Allocates once per
 * context; without it embla_attn_full_prefill runs every unit as one CTA. Call it at set-up: the attention calls
 * themselves never allocate or synchronise. */
EmblaStatus embla_attn_reserve_prefill(EmblaAttn* ctx, void* stream);

/* ---- one decode step through a stack of layers ------------------------------------------------------- */
/* The attention half of Engine.encodeStep's per-layer loop (Engine.swift:933-991 calling
 * encodeAttention, :743-832) as one call: for every layer, the KV write of the current token and the
 * layer's attention, enqueued on one stream. */
enum {   /* Embla.Kind, Engine.swift:14; a sparse layer either owns 16-bit keys (SPARSE) or, as in the reference,
            reads the preceding full layer's int8 cache (SPARSE_SHARED, Engine.swift:461-462) */
    EMBLA_LAYER_SLIDING = 0, EMBLA_LAYER_FULL = 1, EMBLA_LAYER_SPARSE = 2, EMBLA_LAYER_SPARSE_SHARED = 3
};
enum {   /* entry points a step launches, for embla_stack_set_probe */
    EMBLA_ENTRY_APPEND = 0, EMBLA_ENTRY_FULL_DECODE = 1, EMBLA_ENTRY_SLIDING_WRITE = 2, EMBLA_ENTRY_SLIDING_DECODE = 3,
    EMBLA_ENTRY_SCORE = 4, EMBLA_ENTRY_SELECT = 5, EMBLA_ENTRY_SPARSE_DECODE = 6
};

typedef struct {
    int32_t     kind;        /* EMBLA_LAYER_* */
    int32_t     slot;        /* full: layer of the int8 pool; sparse: layer of the 16-bit pool; sparse shared: the int8
                                pool layer of the full layer whose cache it reads; sliding: ring index */
    int32_t     norm_k;      /* full/sparse: RMS-norm k before it is stored (the reference does) */
    int32_t     emit_scores; /* full: 1 = past 1152 keys also write key scores and select rows for the sparse layers
                                that follow (Embla.selects, Engine.swift:24-26, 797) */
    const void* g1_dev;      /* query gains; NULL = queries arrive prenormed (sparse layers: must be NULL) */
    const void* g2_dev;
    const void* kgain_dev;   /* sliding: key gain; NULL = keys arrive prenormed */
} EmblaLayerDesc;

typedef struct {
    const void*    qkv_dev;            /* [n_layers][batch][qkv_stride]: q (n_q_heads*128), k, v (n_kv_heads*128 each) */
    int64_t        qkv_stride;         /* elements between sequences (4096 in the reference) */
    int64_t        qkv_layer_stride;   /* elements between layers */
    void*          o_dev;              /* [n_layers][batch][o_stride] */
    int64_t        o_stride, o_layer_stride;
    const int32_t* seq_lens_dev;       /* [batch] keys visible, the current token included (pos + 1) */
    const int32_t* pos_dev;            /* [batch] position of the current token */
    const int32_t* full_table_dev;     /* block table into the int8 pool */
    int32_t        full_table_stride;
    int32_t        sparse_table_stride;
    const int32_t* sparse_table_dev;   /* block table into the 16-bit pool */
    int32_t        batch;
    int32_t        max_seq_len;        /* host-side upper bound of seq_lens; 0 = max_context */
} EmblaStackStep;

typedef struct EmblaStack EmblaStack;
/* `rings` holds one EmblaRing per sliding layer slot. The pools and rings stay owned by the caller. */
EmblaStatus embla_stack_create(EmblaAttn* ctx, const EmblaLayerDesc* layers, int32_t n_layers, EmblaKVPool* full_pool,
                               EmblaKVPool* sparse_pool, const EmblaRing* rings, int32_t n_rings, EmblaStack** out);
void        embla_stack_destroy(EmblaStack* stack);
EmblaStatus embla_stack_decode_step(EmblaStack* stack, const EmblaStackStep* step, void* stream);
/* The same for layers first_layer .. first_layer + n_layers - 1 only (the step's arrays still hold every layer): a caller
 * whose query rows arrive layer by layer (the q/k/v projections run between the attention layers; a host that feeds them
 * copies them in while earlier layers run) calls this once per group of layers. A sparse layer that shares a full
 * layer's cache and selection must be in a later or the same call as that full layer. */
EmblaStatus embla_stack_decode_layers(EmblaStack* stack, const EmblaStackStep* step, int32_t first_layer, int32_t n_layers,
                                      void* stream);
/* The attention branch of Prefill.encode's per-layer loop (Prefill.swift:282-345) as one call: for a chunk of
 * n_tokens new tokens per sequence at positions pos0_dev[b] + t, every layer of the stack in order:
 *   sliding: kv_sliding_b then attn_sliding(8)_b  -> embla_sliding_write + embla_attn_sliding_prefill
 *   full:    kv_append_b then q_prep_b + relu2_prefill_nax -> embla_kv_append + embla_attn_full_prefill
 * all enqueued on one stream. The last `kv_only_layers` layers of the stack only store their keys and values (the
 * reference's layer 16, "its K/V only", Prefill.swift:286, 327); their rows of o_dev are left untouched. Sparse layers
 * are refused with EMBLA_UNSUPPORTED: the reference's prefill half has none. With split-KV scratch reserved
 * (embla_attn_reserve_prefill) the call neither allocates nor synchronises. */
typedef struct {
    const void*    qkv_dev;            /* [n_layers][batch][n_tokens][qkv_token_stride]: q, k, v of a token as in a decode step */
    int64_t        qkv_token_stride;   /* elements between tokens (4096 in the reference) */
    int64_t        qkv_seq_stride;     /* elements between sequences */
    int64_t        qkv_layer_stride;   /* elements between layers */
    void*          o_dev;              /* [n_layers][batch][n_tokens][o_token_stride] */
    int64_t        o_token_stride, o_seq_stride, o_layer_stride;
    const int32_t* pos0_dev;           /* [batch] position of each sequence's first new token */
    const int32_t* full_table_dev;     /* block table into the int8 pool */
    int32_t        full_table_stride;
    int32_t        batch;
    int32_t        n_tokens;           /* tokens of the chunk, the same for every sequence */
    int32_t        max_seq_len;        /* host-side upper bound of pos0 + n_tokens; 0 = max_context */
    int32_t        kv_only_layers;     /* trailing layers that only store K/V */
} EmblaStackChunk;
EmblaStatus embla_stack_prefill_chunk(EmblaStack* stack, const EmblaStackChunk* chunk, void* stream);
/* Timing probe, the counterpart of the reference's per-part Profiler (StepEncoder.swift:7-65):
 * CUDA events are recorded on the stream around every launch of entry point `entry` (-1: off);
 * read_probe returns their summed time and count since the last read, after the caller has
 * synchronised the stream. */
#define EMBLA_PROBE_FIRST_ONLY 256   /* or-ed into `entry`: only the first launch of that entry point in every step call is
                                        timed (events between two launches keep the second from overlapping the first's
                                        tail, so timing all of them slows the step it measures) */
EmblaStatus embla_stack_set_probe(EmblaStack* stack, int32_t entry);
EmblaStatus embla_stack_read_probe(EmblaStack* stack, float* total_ms, int32_t* launches);

/* ---- Prefix-cache store ---------------------------------------------------------------------------
 * Replaces PrefixCache (Sources/EmblaMetal/PrefixCache.swift:24-145) and Engine.restoreFromStore /
 * saveToStore with their span copies (PrefixCache.swift:150-286; resume rules Engine.swift:346-373).
 * Same index: blocks of 128 positions known by an FNV-1a hash chained over every token before them,
 * a parent/child tree, window checkpoints only at turn ends, least recently used leaves evicted
 * first. A stored block is one contiguous copy of a physical block of the full layers' pool; a
 * checkpoint is the 128 ring slots of every sliding layer (K and V, every kv head), gathered by one
 * launch. The reference's checkpoint also holds 16 rows of engram conv history: not part of this
 * library. All calls on one store must use one stream (a slot freed by an eviction may be refilled
 * by the next save, ordered on that stream). Not thread-safe, as the reference's is not. */
typedef struct EmblaPrefixStore EmblaPrefixStore;
typedef struct {
    int64_t limit_bytes;   /* PrefixCache.limit: most bytes to hold; 0 stores nothing */
    int32_t turn_margin;   /* PrefixCache.turnMargin (16): a turn's checkpoint is at least this far before its end */
    int32_t dry_run;       /* 1: the index only - no device memory, no copies (host-side tests) */
} EmblaPrefixConfig;
/* The caches of one sequence: its row of the full layers' block table (host copy) and its rings. */
typedef struct {
    const EmblaKVPool* pool;              /* the full layers' pool (NULL in a dry run) */
    const int32_t*     block_table_host;  /* physical block of positions 128 i .. 128 i + 127 */
    int32_t            table_len;
    const EmblaRing*   rings;             /* one per sliding layer */
    int32_t            n_rings;
    int32_t            n_kv_heads;        /* of the rings */
    int32_t            ring_slots;        /* Engine.ring: slots of every ring, a multiple of 128 */
    int32_t            seq;               /* the sequence's index in the rings */
} EmblaSeqCaches;

/* PrefixCache.hash (PrefixCache.swift:69-79): FNV-1a over the 4 bytes of every token, little end first, from parent ^ basis. */
uint64_t    embla_prefix_hash(uint64_t parent, const int32_t* tokens, int32_t n);
/* full_block_bytes = embla_kv_block_bytes(pool); window_bytes = n_rings * 2 * n_kv_heads * 128 * 256. */
EmblaStatus embla_prefix_store_create(const EmblaPrefixConfig* cfg, int64_t full_block_bytes, int64_t window_bytes,
                                      EmblaPrefixStore** out);
void        embla_prefix_store_destroy(EmblaPrefixStore* store);
void        embla_prefix_store_remove_all(EmblaPrefixStore* store);
EmblaStatus embla_prefix_store_stats(const EmblaPrefixStore* store, int64_t* bytes, int32_t* blocks, int32_t* checkpoints,
                                     int64_t* evicted);
/* PrefixCache.chain: how many stored blocks `tokens` starts with, covering at most up_to positions; the first
 * `cap` of their hashes and checkpoint flags are written when the pointers are not NULL. */
int32_t     embla_prefix_store_chain(const EmblaPrefixStore* store, const int32_t* tokens, int32_t n_tokens, int32_t up_to,
                                     uint64_t* hashes_out, int32_t* has_window_out, int32_t cap);
/* Engine.restoreFromStore: if the last checkpoint block the prompt starts with ends beyond `reuse` (where the live
 * caches can resume), copies that checkpoint into the rings and the stored blocks ending beyond `live` into the
 * physical blocks of dst's table, and returns its end in *start_out (and start - 128 in *ring_valid_from_out);
 * else *start_out = -1. */
EmblaStatus embla_prefix_store_restore(EmblaPrefixStore* store, const EmblaSeqCaches* dst, const int32_t* prompt,
                                       int32_t n_prompt, int32_t live, int32_t reuse, int32_t* start_out,
                                       int32_t* ring_valid_from_out, void* stream);
/* Engine.saveToStore: stores the blocks of positions 0 .. position - 1 the store lacks, and for each turn end the
 * checkpoint of the last block ending at least turn_margin before it, when the rings still hold it; then evicts. */
EmblaStatus embla_prefix_store_save(EmblaPrefixStore* store, const EmblaSeqCaches* src, const int32_t* tokens,
                                    int32_t position, const int32_t* turn_ends, int32_t n_turn_ends,
                                    int32_t ring_valid_from, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* EMBLA_CUDA_ATTN_H */
