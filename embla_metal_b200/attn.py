"""Host-side binding of libembla_cuda_attn.so (the C ABI in include/embla_cuda_attn.h).

The reference dispatches attention from Swift (Engine.encodeAttention, Sources/EmblaMetal/
Engine.swift:743-832; Prefill.encode, Sources/EmblaMetal/Prefill.swift:265-407). No Swift toolchain
exists where this is built, so this ctypes layer is the tested caller of the C ABI; it keeps the
reference's vocabulary (qkv rows, kv heads, seq_lens = pos + 1, selecting past topk + recent keys).
torch is used for device memory and streams only. There is no CPU fallback: if the CUDA library is
missing, importing `lib()` raises.
"""
import ctypes as C
import os

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libembla_cuda_attn.so")

BF16, F16 = 0, 1
KV_INT8, KV_16BIT = 0, 1
SCALE_F32, SCALE_F16 = 0, 1
HEAD_DIM, BLOCK, TOPK, RECENT = 128, 128, 1024, 128
OK, BAD_ARG, OOM, CUDA_ERR, NCCL_ERR, TIMEOUT, UNSUPPORTED = range(7)

_TORCH_DT = {BF16: torch.bfloat16, F16: torch.float16}


class EmblaError(RuntimeError):
    def __init__(self, status, msg):
        super().__init__(f"embla status {status}: {msg}")
        self.status = status


class AttnConfig(C.Structure):
    _fields_ = [("n_q_heads", C.c_int32), ("n_kv_heads", C.c_int32), ("act_dtype", C.c_int32),
                ("max_batch", C.c_int32), ("max_context", C.c_int32)]


class Query(C.Structure):
    _fields_ = [("q_dev", C.c_void_p), ("q_stride", C.c_int64), ("prenormed", C.c_int32), ("ng", C.c_int32),
                ("g1_dev", C.c_void_p), ("g2_dev", C.c_void_p)]


class W4Matrix(C.Structure):
    _fields_ = [("words_dev", C.c_void_p), ("scales_dev", C.c_void_p), ("biases_dev", C.c_void_p), ("rows", C.c_int32)]


class W4Weights:
    """One 4-bit matrix on the device in the reference's layout: words int32 [rows, d_in / 32, 4], scales and biases
    bfloat16 [rows, d_in / 64]."""

    def __init__(self, words, scales, biases):
        self.words, self.scales, self.biases = words.contiguous(), scales.contiguous(), biases.contiguous()
        self.rows, self.d_in = self.words.shape[0], self.words.shape[1] * 32
        self.desc = W4Matrix(self.words.data_ptr(), self.scales.data_ptr(), self.biases.data_ptr(), self.rows)


class KVView(C.Structure):
    _fields_ = [("block_table_dev", C.c_void_p), ("table_stride", C.c_int32), ("seq_lens_dev", C.c_void_p),
                ("batch", C.c_int32), ("layer", C.c_int32), ("max_seq_len", C.c_int32)]


_lib = None


def lib():
    """The loaded CUDA library; raises if it has not been built (no fallback exists)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: run `python -m embla_metal_b200.build` (needs nvcc)")
        L = C.CDLL(LIB_PATH)
        L.embla_version.restype = C.c_char_p
        L.embla_last_error.restype = C.c_char_p
        L.embla_kv_block_bytes.restype = C.c_size_t
        L.embla_kv_page_bytes.restype = C.c_size_t
        L.embla_kv_pool_base.restype = C.c_void_p
        for name in ("embla_kv_block_bytes", "embla_kv_page_bytes", "embla_kv_pool_base", "embla_kv_pool_destroy",
                     "embla_attn_destroy"):
            getattr(L, name).argtypes = [C.c_void_p]
        _lib = L
    return _lib


def _check(status):
    if status != OK:
        raise EmblaError(status, lib().embla_last_error().decode())


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


class KVPool:
    """Paged KV pool of 128-position blocks (the full layers' cache of Engine.swift:269-284)."""

    def __init__(self, n_layers, n_kv_heads, num_blocks, kv_dtype=KV_INT8, scale_dtype=SCALE_F16):
        self.handle = C.c_void_p()
        _check(lib().embla_kv_pool_create(n_layers, n_kv_heads, kv_dtype, scale_dtype, num_blocks, C.byref(self.handle)))
        self.n_layers, self.n_kv_heads, self.num_blocks = n_layers, n_kv_heads, num_blocks
        self.kv_dtype, self.scale_dtype = kv_dtype, scale_dtype
        self.block_bytes = lib().embla_kv_block_bytes(self.handle)
        self.page_bytes = lib().embla_kv_page_bytes(self.handle)

    def close(self):
        if self.handle:
            lib().embla_kv_pool_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:   # interpreter shutdown
            pass

    def raw(self):
        """The pool as a uint8 tensor [num_blocks, n_layers, n_kv_heads, page_bytes] aliasing device memory."""
        base = lib().embla_kv_pool_base(self.handle)
        shape = (self.num_blocks, self.n_layers, self.n_kv_heads, self.page_bytes)

        class _Dev:
            __cuda_array_interface__ = {"shape": shape, "typestr": "|u1", "data": (base, False), "version": 3}

        self._keep = _Dev()
        return torch.as_tensor(self._keep, device="cuda")

    def export_block(self, block, dst):
        _check(lib().embla_kv_block_export(self.handle, block, _ptr(dst), _stream()))

    def import_block(self, block, src):
        _check(lib().embla_kv_block_import(self.handle, block, _ptr(src), _stream()))


class Attention:
    """Context of the attention path: shape, activation dtype, split-K scratch."""

    def __init__(self, n_q_heads=16, n_kv_heads=4, act_dtype=F16, max_batch=1, max_context=32768):
        self.cfg = AttnConfig(n_q_heads, n_kv_heads, act_dtype, max_batch, max_context)
        self.handle = C.c_void_p()
        _check(lib().embla_attn_create(C.byref(self.cfg), C.byref(self.handle)))
        self.torch_dtype = _TORCH_DT[act_dtype]

    def close(self):
        if self.handle:
            lib().embla_attn_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:   # interpreter shutdown
            pass

    def check(self):
        _check(lib().embla_attn_check(self.handle, _stream()))

    def set_wait_limit(self, cycles):
        """Bound of the device-side waits of this context's launches, in SM clocks."""
        _check(lib().embla_attn_set_wait_limit(self.handle, C.c_int64(cycles)))

    STALL_PARTIALS = 1 << 30   # EMBLA_STALL_PARTIALS

    def inject_stall(self, item):
        """Diagnostic: producers stop requesting data at `item` of their range (None or -1: off)."""
        _check(lib().embla_attn_inject_stall(self.handle, -1 if item is None else int(item)))

    def trace_begin(self, max_launches=256):
        _check(lib().embla_attn_trace_begin(self.handle, max_launches, _stream()))
        self._trace_cap = max_launches

    def trace_end(self):
        """[(entry, first_enter_ns, first_ready_ns, last_loop_end_ns, last_exit_ns, 4 phase marks)] of the launches since
        trace_begin."""
        cap = self._trace_cap
        stamps = (C.c_uint64 * (8 * cap))()
        entries = (C.c_int32 * cap)()
        n = C.c_int32()
        _check(lib().embla_attn_trace_end(self.handle, _stream(), stamps, entries, cap, C.byref(n)))
        return [(entries[i], *[stamps[8 * i + k] for k in range(8)]) for i in range(n.value)]

    @staticmethod
    def view(block_table, seq_lens, layer, max_seq_len=0):
        return KVView(block_table.data_ptr(), block_table.stride(0), None if seq_lens is None else seq_lens.data_ptr(),
                      block_table.shape[0], layer, max_seq_len)

    @staticmethod
    def query(q, gains=None):
        """q [batch, >= n_q_heads * 128] (row stride = the tensor's); gains = (g1, g2) or None (prenormed)."""
        if gains is None:
            return Query(q.data_ptr(), q.stride(0), 1, 0, None, None)
        g1, g2 = gains
        ng = 2 if g2 is not None else 1
        return Query(q.data_ptr(), q.stride(0), 0, ng, g1.data_ptr(), None if g2 is None else g2.data_ptr())

    def qkv_project(self, wq, wk, wv, x, qkv):
        """qkv [batch, >= (Hq + 2 Hkv) * 128] <- the 4-bit GEMVs of x [batch, d_in] (W4Weights), rounded to the dtype."""
        _check(lib().embla_qkv_project(self.handle, C.byref(wq.desc), C.byref(wk.desc), C.byref(wv.desc), wq.d_in, _ptr(x),
                                       C.c_int64(x.stride(0)), x.shape[0], _ptr(qkv), C.c_int64(qkv.stride(0)), _stream()))

    def qkv_project_full_step(self, wq, wk, wv, x, qkv, pool, block_table, seq_lens, layer, gains=None, norm_k=True):
        """The same with the full layer's epilogue: q head-normed with `gains` into qkv (prenormed for full_decode), the
        token's k and v quantised into the int8 pool at position seq_len - 1."""
        view = self.view(block_table, seq_lens, layer)
        qd = self.query(qkv, gains)
        _check(lib().embla_qkv_project_full_step(self.handle, C.byref(wq.desc), C.byref(wk.desc), C.byref(wv.desc), wq.d_in, _ptr(x),
                                                 C.c_int64(x.stride(0)), C.byref(qd), pool.handle, C.byref(view), int(norm_k),
                                                 _ptr(qkv), C.c_int64(qkv.stride(0)), _stream()))

    def qkv_project_sliding_step(self, wq, wk, wv, x, qkv, ring, seq_lens, qgain=None, kgain=None):
        """The producer for a sliding layer: q normed with qgain and rotated into qkv (prenormed for sliding_decode), the
        token's k (normed with kgain, rotated) and v written to the ring slot of position seq_len - 1."""
        _check(lib().embla_qkv_project_sliding_step(self.handle, C.byref(wq.desc), C.byref(wk.desc), C.byref(wv.desc), wq.d_in,
                                                    _ptr(x), C.c_int64(x.stride(0)), _ptr(qgain), _ptr(kgain), C.byref(ring.desc),
                                                    _ptr(seq_lens), x.shape[0], _ptr(qkv), C.c_int64(qkv.stride(0)), _stream()))

    def oproj(self, wo, o, x, accumulate=True):
        """x fp32 [batch, >= rows] (+)= the 4-bit GEMV of the attention output rows o [batch, d_in], rounded to the dtype."""
        _check(lib().embla_oproj(self.handle, C.byref(wo.desc), wo.d_in, _ptr(o), C.c_int64(o.stride(0)), o.shape[0], _ptr(x),
                                 C.c_int64(x.stride(0)), int(accumulate), _stream()))

    def kv_append(self, pool, block_table, layer, pos0, k, v, norm_k=True):
        """k, v [batch, n_tokens, n_kv_heads * 128 (or wider rows)]; pos0 int32 [batch] first position."""
        view = self.view(block_table, None, layer)
        _check(lib().embla_kv_append(self.handle, pool.handle, C.byref(view), _ptr(pos0), k.shape[1], _ptr(k), _ptr(v),
                                     C.c_int64(k.stride(1)), C.c_int64(k.stride(0)), int(norm_k), _stream()))

    def full_decode(self, pool, block_table, seq_lens, layer, q, o, gains=None, scores=None, max_seq_len=0):
        view = self.view(block_table, seq_lens, layer, max_seq_len)
        qd = self.query(q, gains)
        _check(lib().embla_attn_full_decode(self.handle, pool.handle, C.byref(view), C.byref(qd), _ptr(o),
                                            C.c_int64(o.stride(0)), _ptr(scores),
                                            C.c_int64(0 if scores is None else scores.stride(1)), _stream()))

    def score_keys(self, pool, block_table, seq_lens, layer, q, scores, max_seq_len=0):
        """scores [batch, n_kv_heads, >= max_seq_len] fp32 <- max over the kv head's query heads of q·k."""
        view = self.view(block_table, seq_lens, layer, max_seq_len)
        _check(lib().embla_score_keys(self.handle, pool.handle, C.byref(view), _ptr(q), C.c_int64(q.stride(0)),
                                      _ptr(scores), C.c_int64(scores.stride(1)), _stream()))

    def full_step(self, pool, block_table, seq_lens, layer, q, k, v, o, gains=None, scores=None, max_seq_len=0, norm_k=True):
        """kv_append of the current token (k, v [batch, >= n_kv_heads * 128]) and full_decode in one launch."""
        view = self.view(block_table, seq_lens, layer, max_seq_len)
        qd = self.query(q, gains)
        _check(lib().embla_attn_full_step(self.handle, pool.handle, C.byref(view), C.byref(qd), _ptr(k), _ptr(v),
                                          C.c_int64(k.stride(0)), int(norm_k), _ptr(o), C.c_int64(o.stride(0)), _ptr(scores),
                                          C.c_int64(0 if scores is None else scores.stride(1)), _stream()))

    def score_keys_step(self, pool, block_table, seq_lens, layer, q, k, v, scores, max_seq_len=0, norm_k=True):
        """kv_append of the current token into the 16-bit pool and score_keys in one launch."""
        view = self.view(block_table, seq_lens, layer, max_seq_len)
        _check(lib().embla_score_keys_step(self.handle, pool.handle, C.byref(view), _ptr(q), C.c_int64(q.stride(0)), _ptr(k), _ptr(v),
                                           C.c_int64(k.stride(0)), int(norm_k), _ptr(scores), C.c_int64(scores.stride(1)), _stream()))

    def select_keys(self, scores, seq_lens, idx, max_seq_len=0):
        """idx [batch, n_kv_heads, 1152] uint32 (int32 tensor) <- top 1024 + 128 latest per kv head."""
        _check(lib().embla_select_keys(self.handle, _ptr(scores), C.c_int64(scores.stride(1)), _ptr(seq_lens),
                                       scores.shape[0], max_seq_len, _ptr(idx), _stream()))

    def sparse_decode(self, pool, block_table, seq_lens, layer, q, o, idx=None, gains=None, max_seq_len=0):
        view = self.view(block_table, seq_lens, layer, max_seq_len)
        qd = self.query(q, gains)
        _check(lib().embla_attn_sparse_decode(self.handle, pool.handle, C.byref(view), C.byref(qd), _ptr(idx), _ptr(o),
                                              C.c_int64(o.stride(0)), _stream()))

    def sliding_write(self, ring, pos0, k, v, kgain=None):
        """k, v [batch, n_tokens, n_kv_heads * 128 (or wider rows)] into the rings at positions pos0[b] + t."""
        _check(lib().embla_sliding_write(self.handle, C.byref(ring.desc), _ptr(pos0), k.shape[0], k.shape[1], _ptr(k),
                                         _ptr(v), C.c_int64(k.stride(1)), C.c_int64(k.stride(0)), int(kgain is None),
                                         _ptr(kgain), _stream()))

    def sliding_decode(self, ring, seq_lens, q, o, qgain=None):
        qd = self.query(q, None if qgain is None else (qgain, None))
        _check(lib().embla_attn_sliding_decode(self.handle, C.byref(ring.desc), _ptr(seq_lens), q.shape[0], C.byref(qd),
                                               _ptr(o), C.c_int64(o.stride(0)), _stream()))


class RingDesc(C.Structure):
    _fields_ = [("k_dev", C.c_void_p), ("v_dev", C.c_void_p), ("seq_stride", C.c_int64), ("ring", C.c_int32),
                ("window", C.c_int32)]


class Ring:
    """Sliding-layer rings of a batch: k, v [batch, n_kv_heads, ring, 128] in the activation dtype."""

    def __init__(self, batch, n_kv_heads, ring, window, torch_dtype):
        self.k = torch.zeros(batch, n_kv_heads, ring, HEAD_DIM, dtype=torch_dtype, device="cuda")
        self.v = torch.zeros_like(self.k)
        self.desc = RingDesc(self.k.data_ptr(), self.v.data_ptr(), self.k.stride(0), ring, window)


def full_prefill(ctx, pool, block_table, layer, pos0, q, o, gains=None, qk8=False):
    """Causal ReLU² attention of a prefill chunk. q [batch, n_tokens, >= n_q_heads*128], o likewise
    (token-major); pos0 int32 [batch]. The chunk's keys/values must already be appended. qk8: the int8 Q Kᵀ
    build (embla_attn_full_prefill_qk8)."""
    view = Attention.view(block_table, None, layer)
    if gains is None:
        qd = Query(q.data_ptr(), q.stride(0), 1, 0, None, None)
    else:
        qd = Query(q.data_ptr(), q.stride(0), 0, 2, gains[0].data_ptr(), gains[1].data_ptr())
    if not getattr(ctx, "_prefill_reserved", False):   # set-up, once per context: the split-KV scratch
        _check(lib().embla_attn_reserve_prefill(ctx.handle, _stream()))
        ctx._prefill_reserved = True
    fn = lib().embla_attn_full_prefill_qk8 if qk8 else lib().embla_attn_full_prefill
    _check(fn(ctx.handle, pool.handle, C.byref(view), _ptr(pos0), q.shape[1], C.byref(qd),
              C.c_int64(q.stride(1)), _ptr(o), C.c_int64(o.stride(1)), C.c_int64(o.stride(0)), _stream()))


def full_prefill_scatter(ctx, pool, block_table, layer, pos0, q, o, peer_ptrs, o_token_stride, gains=None):
    """embla_attn_full_prefill that also stores its rows to `peer_ptrs` (device addresses in other GPUs' memory: where this
    rank's slab starts inside each GPU's token-major output, rows `o_token_stride` elements apart). o [1, n_tokens, ...]
    is this GPU's own place of the slab, a view with the same row stride."""
    view = Attention.view(block_table, None, layer)
    if gains is None:
        qd = Query(q.data_ptr(), q.stride(0), 1, 0, None, None)
    else:
        qd = Query(q.data_ptr(), q.stride(0), 0, 2, gains[0].data_ptr(), gains[1].data_ptr())
    if not getattr(ctx, "_prefill_reserved", False):
        _check(lib().embla_attn_reserve_prefill(ctx.handle, _stream()))
        ctx._prefill_reserved = True
    arr = (C.c_void_p * max(1, len(peer_ptrs)))(*[C.c_void_p(p) for p in peer_ptrs])
    _check(lib().embla_attn_full_prefill_scatter(ctx.handle, pool.handle, C.byref(view), _ptr(pos0), q.shape[1], C.byref(qd),
                                                 C.c_int64(q.stride(1)), _ptr(o), arr, len(peer_ptrs), C.c_int64(o_token_stride),
                                                 C.c_int64(o.stride(0)), _stream()))


def sliding_prefill(ctx, ring, pos0, q, o, qgain=None):
    """Softmax attention of a prefill chunk over each token's window; q, o [batch, n_tokens, >= n_q_heads*128].
    The chunk's keys/values must already be in the ring (Attention.sliding_write)."""
    if qgain is None:
        qd = Query(q.data_ptr(), q.stride(0), 1, 0, None, None)
    else:
        qd = Query(q.data_ptr(), q.stride(0), 0, 1, qgain.data_ptr(), None)
    _check(lib().embla_attn_sliding_prefill(ctx.handle, C.byref(ring.desc), _ptr(pos0), q.shape[0], q.shape[1], C.byref(qd),
                                            C.c_int64(q.stride(1)), _ptr(o), C.c_int64(o.stride(1)), C.c_int64(o.stride(0)),
                                            _stream()))
