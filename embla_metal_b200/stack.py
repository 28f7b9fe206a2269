"""A stack of attention layers decoding one token per sequence: binding of embla_stack_* (the
attention half of the reference's Engine.encodeStep loop, Sources/EmblaMetal/Engine.swift:933-991).

`DecodeStack` owns the KV state of a batch of sequences — the int8 pool of the full layers, the
16-bit pool of the sparse layers, the sliding layers' rings, and identity block tables — and runs a
step from device-resident `qkv` rows or, through `step_host`, from pinned host buffers.
"""
import ctypes as C

import torch

from . import attn

SLIDING, FULL, SPARSE, SPARSE_SHARED = 0, 1, 2, 3
ENTRY = {"append": 0, "full_decode": 1, "sliding_write": 2, "sliding_decode": 3, "score": 4, "select": 5,
         "sparse_decode": 6}


class LayerDesc(C.Structure):
    _fields_ = [("kind", C.c_int32), ("slot", C.c_int32), ("norm_k", C.c_int32), ("emit_scores", C.c_int32),
                ("g1_dev", C.c_void_p), ("g2_dev", C.c_void_p), ("kgain_dev", C.c_void_p)]


class StackStep(C.Structure):
    _fields_ = [("qkv_dev", C.c_void_p), ("qkv_stride", C.c_int64), ("qkv_layer_stride", C.c_int64),
                ("o_dev", C.c_void_p), ("o_stride", C.c_int64), ("o_layer_stride", C.c_int64),
                ("seq_lens_dev", C.c_void_p), ("pos_dev", C.c_void_p), ("full_table_dev", C.c_void_p),
                ("full_table_stride", C.c_int32), ("sparse_table_stride", C.c_int32), ("sparse_table_dev", C.c_void_p),
                ("batch", C.c_int32), ("max_seq_len", C.c_int32)]


class StackChunk(C.Structure):
    _fields_ = [("qkv_dev", C.c_void_p), ("qkv_token_stride", C.c_int64), ("qkv_seq_stride", C.c_int64),
                ("qkv_layer_stride", C.c_int64), ("o_dev", C.c_void_p), ("o_token_stride", C.c_int64),
                ("o_seq_stride", C.c_int64), ("o_layer_stride", C.c_int64), ("pos0_dev", C.c_void_p),
                ("full_table_dev", C.c_void_p), ("full_table_stride", C.c_int32), ("batch", C.c_int32),
                ("n_tokens", C.c_int32), ("max_seq_len", C.c_int32), ("kv_only_layers", C.c_int32)]


def cycle_kinds(n_layers):
    """The benchmark's stack: layers cycling sparse, sliding, sliding, full."""
    return [(SPARSE, SLIDING, SLIDING, FULL)[i % 4] for i in range(n_layers)]


class DecodeStack:
    def __init__(self, kinds, batch, max_context, n_q_heads=16, n_kv_heads=4, act_dtype=attn.F16, window=1024,
                 ring=4096, scale_dtype=attn.SCALE_F16, norm_k=False):
        self.kinds, self.batch, self.max_context = list(kinds), batch, max_context
        self.Hq, self.Hkv = n_q_heads, n_kv_heads
        self.ctx = attn.Attention(n_q_heads, n_kv_heads, act_dtype, max_batch=batch, max_context=max_context)
        self.dtype = self.ctx.torch_dtype
        npages = (max_context + attn.BLOCK - 1) // attn.BLOCK
        self.npages = npages
        n_full = sum(k == FULL for k in self.kinds)
        n_sparse = sum(k == SPARSE for k in self.kinds)
        n_sliding = sum(k == SLIDING for k in self.kinds)
        self.full_pool = attn.KVPool(n_full, n_kv_heads, batch * npages, attn.KV_INT8, scale_dtype) if n_full else None
        self.sparse_pool = attn.KVPool(n_sparse, n_kv_heads, batch * npages, attn.KV_16BIT) if n_sparse else None
        self.rings = [attn.Ring(batch, n_kv_heads, ring, window, self.dtype) for _ in range(n_sliding)]
        # sequence b owns blocks b * npages .. of each pool
        self.table = torch.arange(batch * npages, dtype=torch.int32, device="cuda").view(batch, npages).contiguous()
        descs = (LayerDesc * len(self.kinds))()
        slots = {SLIDING: 0, FULL: 0, SPARSE: 0}
        for i, k in enumerate(self.kinds):
            if k == SPARSE_SHARED:
                # reads the cache of the closest preceding full layer (Embla.blockFull, Engine.swift:22)
                if slots[FULL] == 0:
                    raise ValueError("a sparse layer that shares a cache needs a full layer before it")
                descs[i] = LayerDesc(k, slots[FULL] - 1, 0, 0, None, None, None)
                continue
            shared_next = k == FULL and i + 1 < len(self.kinds) and self.kinds[i + 1] == SPARSE_SHARED
            descs[i] = LayerDesc(k, slots[k], int(norm_k), int(shared_next), None, None, None)
            slots[k] += 1
        ring_descs = (attn.RingDesc * max(1, n_sliding))()
        for i, r in enumerate(self.rings):
            ring_descs[i] = r.desc
        self.handle = C.c_void_p()
        L = attn.lib()
        attn._check(L.embla_stack_create(self.ctx.handle, descs, len(self.kinds),
                                         self.full_pool.handle if self.full_pool else None,
                                         self.sparse_pool.handle if self.sparse_pool else None,
                                         ring_descs, n_sliding, C.byref(self.handle)))
        self.qkv_width = (n_q_heads + 2 * n_kv_heads) * attn.HEAD_DIM
        self.o_width = n_q_heads * attn.HEAD_DIM
        n = len(self.kinds)
        self.qkv = torch.zeros(n, batch, self.qkv_width, dtype=self.dtype, device="cuda")
        self.o = torch.zeros(n, batch, self.o_width, dtype=self.dtype, device="cuda")
        self.qkv_host = torch.zeros(n, batch, self.qkv_width, dtype=self.dtype).pin_memory()
        self.o_host = torch.zeros(n, batch, self.o_width, dtype=self.dtype).pin_memory()
        self.seq_lens = torch.zeros(batch, dtype=torch.int32, device="cuda")
        self.pos = torch.zeros(batch, dtype=torch.int32, device="cuda")
        self.max_seq_len = max_context

    def close(self):
        if self.handle:
            attn.lib().embla_stack_destroy(self.handle)
            self.handle = C.c_void_p()
        for obj in (self.full_pool, self.sparse_pool, self.ctx):
            if obj is not None:
                obj.close()

    def set_positions(self, pos):
        """pos: int or list — position of the token each sequence decodes next (keys seen = pos + 1)."""
        t = torch.as_tensor([pos] * self.batch if isinstance(pos, int) else list(pos), dtype=torch.int32)
        self.pos.copy_(t)
        self.seq_lens.copy_(t + 1)
        self.max_seq_len = int(t.max()) + 1

    def fill_random(self, seed=0):
        """Synthetic KV state in the benchmark's distributions: int8 codes uniform in [-127, 127] with fp16
        scales uniform in [0.005, 0.02]; 16-bit keys/values ~ N(0, 1) with 1 % of the keys scaled x4."""
        g = torch.Generator(device="cuda").manual_seed(seed)
        if self.full_pool is not None:
            raw = self.full_pool.raw()
            flat = raw.view(-1, raw.shape[-1])
            step = max(1, (1 << 28) // flat.shape[1])
            sdt = torch.float16 if self.full_pool.scale_dtype == attn.SCALE_F16 else torch.float32
            for i in range(0, flat.shape[0], step):
                part = flat[i:i + step]
                codes = torch.randint(-127, 128, (part.shape[0], 32768), dtype=torch.int8, device="cuda", generator=g)
                part[:, :32768] = codes.view(torch.uint8)
                sc = torch.empty(part.shape[0], 256, device="cuda").uniform_(0.005, 0.02, generator=g).to(sdt)
                part[:, 32768:] = sc.view(torch.uint8)
        if self.sparse_pool is not None:
            raw = self.sparse_pool.raw()
            flat = raw.view(-1, raw.shape[-1]).view(self.dtype)       # [pages, 2 * 128 * 128]
            step = max(1, (1 << 27) // flat.shape[1])
            for i in range(0, flat.shape[0], step):
                part = flat[i:i + step]
                vals = torch.randn(part.shape, device="cuda", generator=g)
                keys = vals[:, :16384].view(part.shape[0], 128, 128)
                boost = torch.rand(part.shape[0], 128, 1, device="cuda", generator=g) < 0.01
                keys.mul_(torch.where(boost, 4.0, 1.0))
                part.copy_(vals.to(self.dtype))
        for r in self.rings:
            r.k.copy_(torch.randn(r.k.shape, device="cuda", generator=g).to(self.dtype))
            r.v.copy_(torch.randn(r.v.shape, device="cuda", generator=g).to(self.dtype))

    def _step_struct(self):
        return StackStep(self.qkv.data_ptr(), self.qkv.stride(1), self.qkv.stride(0), self.o.data_ptr(),
                         self.o.stride(1), self.o.stride(0), self.seq_lens.data_ptr(), self.pos.data_ptr(),
                         self.table.data_ptr(), self.table.stride(0), self.table.stride(0), self.table.data_ptr(),
                         self.batch, self.max_seq_len)

    def step(self):
        """One decode step from the device-resident qkv rows; results in self.o."""
        st = self._step_struct()
        attn._check(attn.lib().embla_stack_decode_step(self.handle, C.byref(st), attn._stream()))

    def prefill_chunk(self, qkv, o, pos0, kv_only_layers=0, max_seq_len=0):
        """A chunk of new tokens through every layer (sliding and full layers only): qkv [n_layers, batch, T, qkv_width],
        o [n_layers, batch, T, o_width] on the device, pos0 int32 [batch] the position of each sequence's first new token.
        The last `kv_only_layers` layers only store their keys and values."""
        n, b, t, _ = qkv.shape
        if (n, b) != (len(self.kinds), self.batch) or tuple(o.shape[:3]) != (n, b, t):
            raise ValueError(f"qkv {tuple(qkv.shape)} / o {tuple(o.shape)} do not fit {len(self.kinds)} layers x {self.batch} sequences")
        if qkv.stride(3) != 1 or o.stride(3) != 1:
            raise ValueError("rows must be contiguous")
        ck = StackChunk(qkv.data_ptr(), qkv.stride(2), qkv.stride(1), qkv.stride(0), o.data_ptr(), o.stride(2), o.stride(1),
                        o.stride(0), pos0.data_ptr(), self.table.data_ptr(), self.table.stride(0), b, t, max_seq_len, kv_only_layers)
        attn._check(attn.lib().embla_stack_prefill_chunk(self.handle, C.byref(ck), attn._stream()))

    def step_layers(self, first, count):
        """The step for layers first .. first + count - 1 only."""
        st = self._step_struct()
        attn._check(attn.lib().embla_stack_decode_layers(self.handle, C.byref(st), first, count, attn._stream()))

    def step_host(self, group=4):
        """One decode step from pinned host rows: qkv_host -> device, attention, o -> o_host. The rows travel in groups of
        `group` layers on two copy streams of their own, so a group's rows arrive while the groups before it are attended
        and its outputs leave while the groups after it run; the calling stream ends up behind all of it (a synchronize
        on it, or an event recorded on it, covers the outputs in o_host). group=0: one copy in, the step, one copy out."""
        if not group:
            self.qkv.copy_(self.qkv_host, non_blocking=True)
            self.step()
            self.o_host.copy_(self.o, non_blocking=True)
            return
        cur = torch.cuda.current_stream()
        n = len(self.kinds)
        starts = list(range(0, n, group))
        if getattr(self, "_copy_streams", None) is None:
            self._copy_streams = (torch.cuda.Stream(), torch.cuda.Stream())
            self._copy_events = {}
        if len(self._copy_events.get("in", ())) != len(starts):
            self._copy_events = {"in": [torch.cuda.Event() for _ in starts], "done": [torch.cuda.Event() for _ in starts]}
        s_in, s_out = self._copy_streams
        s_in.wait_stream(cur)          # the step before has read its rows and handed over its outputs
        s_out.wait_stream(cur)
        for i, a in enumerate(starts):
            with torch.cuda.stream(s_in):
                self.qkv[a:a + group].copy_(self.qkv_host[a:a + group], non_blocking=True)
                self._copy_events["in"][i].record(s_in)
        for i, a in enumerate(starts):
            cur.wait_event(self._copy_events["in"][i])
            self.step_layers(a, min(group, n - a))
            self._copy_events["done"][i].record(cur)
            with torch.cuda.stream(s_out):
                s_out.wait_event(self._copy_events["done"][i])
                self.o_host[a:a + group].copy_(self.o[a:a + group], non_blocking=True)
        cur.wait_stream(s_out)

    def set_probe(self, name, first_only=False):
        """Times every launch of entry point `name` (None: off) with events on the stream, or only the first one of every
        step when `first_only` (which leaves the step's other launches overlapping as they do unobserved)."""
        attn._check(attn.lib().embla_stack_set_probe(self.handle, -1 if name is None else ENTRY[name] | (256 if first_only else 0)))

    def read_probe(self):
        ms, n = C.c_float(), C.c_int32()
        attn._check(attn.lib().embla_stack_read_probe(self.handle, C.byref(ms), C.byref(n)))
        return ms.value, n.value

    def launches_per_step(self):
        """Kernels of this library one step launches."""
        selecting = self.max_seq_len > attn.TOPK + attn.RECENT
        per = {SLIDING: 1, FULL: 1, SPARSE: 3 if selecting else 2, SPARSE_SHARED: 1}
        n = sum(per[k] for k in self.kinds)
        if selecting:   # a full layer followed by a shared-cache sparse layer also selects
            n += sum(1 for i, k in enumerate(self.kinds[:-1]) if k == FULL and self.kinds[i + 1] == SPARSE_SHARED)
        return n
