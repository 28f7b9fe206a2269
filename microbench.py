"""Single-kernel timing cases on synthetic data (CUDA events; also the commands profiled under ncu).

    python microbench.py full_decode --batch 8 [--scores]
    python microbench.py sparse --batch 8        # score, select, gather-attend, sliding attend
    python microbench.py prefill --tokens 2048 --cached 30720

Each case prints one line per kernel with its time per launch and the bandwidth or FLOP rate that follows
from the algorithmic bytes / FLOPs of the launch.
"""
import argparse

import torch

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from embla_metal_b200 import attn, stack as stk  # noqa: E402

HQ, HKV, CTX = 16, 4, 32768


def _events(fn, reps=10, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(reps + 1)]
    ev[0].record()
    for i in range(reps):
        fn()
        ev[i + 1].record()
    torch.cuda.synchronize()
    return sorted(ev[i].elapsed_time(ev[i + 1]) for i in range(reps))


def full_decode(batch, scores, kv16=False):
    npg = CTX // 128
    ctx = attn.Attention(HQ, HKV, attn.F16, max_batch=batch, max_context=CTX)
    if kv16:   # the build without the int8 cache: rows in the activation dtype, 512 B a key
        pool = attn.KVPool(1, HKV, batch * npg, attn.KV_16BIT)
        pool.raw().view(torch.float16).normal_()
    else:
        pool = attn.KVPool(1, HKV, batch * npg, attn.KV_INT8, attn.SCALE_F16)
        raw = pool.raw()
        raw.view(-1).random_(0, 256)
        raw[..., 32768:].view(torch.float16).fill_(0.01)
    table = torch.randperm(batch * npg, device="cuda", dtype=torch.int32).view(batch, npg).contiguous()
    lens = torch.full((batch,), CTX, dtype=torch.int32, device="cuda")
    q = torch.randn(batch, HQ * 128, device="cuda", dtype=torch.float16)
    o = torch.zeros_like(q)
    sc = torch.zeros(batch, HKV, CTX, device="cuda") if scores else None
    ts = _events(lambda: ctx.full_decode(pool, table, lens, 0, q, o, scores=sc, max_seq_len=CTX))
    ctx.check()
    nbytes = batch * HKV * CTX * (512 if kv16 else 260)
    print(f"full_decode{' (16-bit cache)' if kv16 else ''} batch {batch} scores {bool(scores)}: {1e3 * ts[len(ts) // 2]:.1f} us/launch, "
          f"{nbytes / ts[len(ts) // 2] / 1e6:.0f} GB/s (min {nbytes / ts[0] / 1e6:.0f})")


def sparse(batch):
    st = stk.DecodeStack([stk.SPARSE, stk.SLIDING], batch, CTX)
    st.fill_random(1)
    st.set_positions(CTX - 1)
    st.qkv.copy_(torch.randn(st.qkv.shape, device="cuda").to(st.dtype))
    for _ in range(3):
        st.step()
    torch.cuda.synchronize()
    pairs = batch * HKV
    nbytes = {"score": pairs * CTX * 256, "select": pairs * (CTX - 128) * 4, "sparse_decode": pairs * 1152 * 512,
              "sliding_decode": pairs * 1024 * 512, "append": pairs * 512, "sliding_write": pairs * 512}
    for name in ("score", "select", "sparse_decode", "sliding_decode", "append", "sliding_write"):
        st.set_probe(name)
        for _ in range(5):
            st.step()
        torch.cuda.synchronize()
        ms, n = st.read_probe()
        if n == 0 or ms == 0.0:
            continue   # not launched by this stack (the sliding ring write is fused into the attention launch)
        print(f"{name} batch {batch}: {1e3 * ms / n:.1f} us/launch, {nbytes[name] / (ms / n) / 1e6:.0f} GB/s")
    st.ctx.check()


def prefill(tokens, cached, qk8=False):
    S = cached + tokens
    npg = (S + 127) // 128
    ctx = attn.Attention(HQ, HKV, attn.BF16, 1, npg * 128)
    pool = attn.KVPool(1, HKV, npg, attn.KV_INT8, attn.SCALE_F16)
    raw = pool.raw()
    raw.view(-1).random_(0, 256)
    raw[..., 32768:].view(torch.float16).fill_(0.01)
    tbl = torch.arange(npg, dtype=torch.int32, device="cuda")[None].contiguous()
    q = torch.randn(1, tokens, HQ * 128, device="cuda", dtype=torch.bfloat16)
    o = torch.zeros_like(q)
    pos0 = torch.tensor([cached], dtype=torch.int32, device="cuda")
    ts = _events(lambda: attn.full_prefill(ctx, pool, tbl, 0, pos0, q, o, qk8=qk8))
    ctx.check()
    flop = 4 * HQ * 128 * sum(cached + i + 1 for i in range(tokens))
    med = ts[len(ts) // 2]
    print(f"full_prefill{' (int8 Q K^T)' if qk8 else ''} {tokens} tokens after {cached}: {med:.4f} ms, {flop / med / 1e9:.0f} TFLOP/s "
          f"(min-time {flop / ts[0] / 1e9:.0f}), {tokens / med * 1e3:.0f} tok/s")


def sliding_prefill(tokens, cached, window, raw=False):
    """Benchmark configuration 1 (b): a chunk of `tokens` appended after `cached` positions of a sliding layer."""
    ring_slots = 4096
    ctx = attn.Attention(HQ, HKV, attn.F16, 1, ring_slots)
    ring = attn.Ring(1, HKV, ring_slots, window, torch.float16)
    ring.k.copy_(torch.randn(ring.k.shape, device="cuda").half())
    ring.v.copy_(torch.randn(ring.v.shape, device="cuda").half())
    q = torch.randn(1, tokens, HQ * 128, device="cuda", dtype=torch.float16)
    o = torch.zeros_like(q)
    pos0 = torch.tensor([cached], dtype=torch.int32, device="cuda")
    gain = (torch.randn(128, device="cuda") * 0.1).half() if raw else None   # raw queries: fused head norm + RoPE
    ts = _events(lambda: attn.sliding_prefill(ctx, ring, pos0, q, o, qgain=gain))
    ctx.check()
    flop = 4 * HQ * 128 * sum(min(cached + i + 1, window) for i in range(tokens))
    med = ts[len(ts) // 2]
    print(f"sliding_prefill {tokens} tokens after {cached}, window {window}: {med:.4f} ms, {flop / med / 1e9:.1f} TFLOP/s, "
          f"{tokens / med * 1e3:.0f} tok/s")


def qkv_project(batch, fused):
    """The q/k/v producer of a full layer: 4-bit GEMV (d_in 2048 -> 16 + 4 + 4 heads of 128) for `batch` tokens."""
    d_in = 2048
    ctx = attn.Attention(HQ, HKV, attn.F16, max_batch=batch, max_context=CTX)
    ws = []
    for rows in (HQ * 128, HKV * 128, HKV * 128):
        words = torch.randint(-2 ** 31, 2 ** 31 - 1, (rows, d_in // 32, 4), dtype=torch.int32, device="cuda")
        sc = torch.full((rows, d_in // 64), 0.005, device="cuda").to(torch.bfloat16).view(torch.int16)
        bs = torch.full((rows, d_in // 64), -0.0375, device="cuda").to(torch.bfloat16).view(torch.int16)
        ws.append(attn.W4Weights(words, sc, bs))
    x = torch.randn(batch, d_in, device="cuda", dtype=torch.float16)
    qkv = torch.zeros(batch, (HQ + 2 * HKV) * 128, device="cuda", dtype=torch.float16)
    npg = CTX // 128
    pool = attn.KVPool(1, HKV, batch * npg, attn.KV_INT8, attn.SCALE_F16)
    table = torch.arange(batch * npg, dtype=torch.int32, device="cuda").view(batch, npg).contiguous()
    lens = torch.full((batch,), CTX, dtype=torch.int32, device="cuda")
    if fused:
        fn = lambda: ctx.qkv_project_full_step(ws[0], ws[1], ws[2], x, qkv, pool, table, lens, 0, norm_k=True)
    else:
        fn = lambda: ctx.qkv_project(ws[0], ws[1], ws[2], x, qkv)
    # the kernel is shorter than a launch from Python: twenty launches replayed from a CUDA graph, timed as one
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(20):
            fn()
    ts = _events(graph.replay)
    ctx.check()
    wbytes = sum(w.words.numel() * 4 + w.scales.numel() * 4 for w in ws)
    print(f"qkv_project batch {batch} fused {bool(fused)}: {1e3 * ts[len(ts) // 2] / 20:.1f} us/launch ({wbytes / 1e6:.1f} MB of weights)")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["full_decode", "sparse", "prefill", "sliding_prefill", "qkv_project"])
    ap.add_argument("--window", type=int, default=1024)
    ap.add_argument("--raw", action="store_true", help="sliding_prefill: queries arrive raw (fused head norm + RoPE)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--scores", action="store_true")
    ap.add_argument("--qk8", action="store_true", help="prefill: the int8 Q K^T build")
    ap.add_argument("--kv16", action="store_true", help="full_decode: a 16-bit cache instead of int8")
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--cached", type=int, default=30720)
    a = ap.parse_args()
    if a.case == "full_decode":
        full_decode(a.batch, a.scores, a.kv16)
    elif a.case == "sparse":
        sparse(a.batch)
    elif a.case == "qkv_project":
        qkv_project(a.batch, a.scores)
    elif a.case == "sliding_prefill":
        sliding_prefill(a.tokens, a.cached if a.cached != 30720 else 2048, a.window, a.raw)
    else:
        prefill(a.tokens, a.cached, a.qk8)


if __name__ == "__main__":
    main()
