#!/usr/bin/env python3
"""Runs the engine's hot kernels alone on the shapes of the Qwen2.5-7B layer, a few launches
each, so that one of them can be captured with ncu (`-k regex:<name>`) or timed.

    python bench_kernels.py [skinny|sgemm|attn_decode|attn_f32|attn_fused|attn_prefill|tc5|tc5_shapes|stream|sample|all] [--once]

Prints the median CUDA-event time and the achieved GB/s or TFLOP/s of each case (a 256 MiB
buffer is written between launches, so every launch starts with a cold L2)."""
import sys

import torch

sys.path.insert(0, __import__("os").path.dirname(__import__("os").path.abspath(__file__)))
from paged_batch_engine_b200.csrc import ops  # noqa: E402

DEV = "cuda:0"
ONCE = "--once" in sys.argv


def timed(fn, flush, n=5):
    if ONCE:                     # under a profiler: one launch of each case is enough
        fn()
        torch.cuda.synchronize()
        return float("nan")
    for _ in range(2):
        fn()
    ts = []
    for _ in range(n):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda._sleep(400000)          # the host enqueues fn() meanwhile: no launch latency in the time
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    return sorted(ts)[len(ts) // 2]


def attention_case(reqs, H=28, KV=4, hd=128, P=16, kind=None, dtype=torch.bfloat16):
    from paged_batch_engine_b200.cache import CacheManager, KVGroupSpec
    from paged_batch_engine_b200.engine.batch import StepContext, StepEntry
    pages = sum((c + n + P - 1) // P for c, n in reqs) + 2
    m = CacheManager([KVGroupSpec((0,), KV, hd)], P, pages, max_requests=len(reqs))
    entries = []
    for c, n in reqs:
        h = m.add_request()
        m.reserve(h, c + n)
        m.commit(h, c)
        entries.append(StepEntry(h, [0] * n))
    kind, tile_rows, _ = ops.attention_kernel_config(hd, dtype, kind)
    key = (0, H // KV, tile_rows, None)
    ctx = StepContext(m, entries, torch.device(DEV), [key])
    meta = ctx.attention_work(0, H // KV, tile_rows, None, H, hd)
    T = sum(n for _, n in reqs)
    q = torch.randn(T, H * hd, device=DEV).to(dtype)
    k = torch.randn(pages, KV, P, hd, device=DEV).to(dtype)
    v = torch.randn(pages, KV, P, hd, device=DEV).to(dtype)
    out = torch.empty_like(q)
    run = lambda: ops.paged_attention(q, k, v, out, meta, H, KV, hd, hd ** -0.5, None, P, kind=kind)
    return run, sum(c + n for c, n in reqs) * KV * hd * 2 * q.element_size()


def fused_decode_case(B, ctx_len, H=28, KV=4, hd=128, P=16):
    """One decoded token a request through the fused kernel (position encoding, cache write,
    attention, merge of the key splits in one launch)."""
    from paged_batch_engine_b200.cache import CacheManager, KVGroupSpec
    from paged_batch_engine_b200.engine.batch import StepContext, StepEntry
    pages = B * ((ctx_len + 1 + P - 1) // P) + 2
    m = CacheManager([KVGroupSpec((0,), KV, hd)], P, pages, max_requests=B)
    entries = []
    for _ in range(B):
        h = m.add_request()
        m.reserve(h, ctx_len + 1)
        m.commit(h, ctx_len)
        entries.append(StepEntry(h, [0]))
    ctx = StepContext(m, entries, torch.device(DEV), [(0, H // KV, 128, None)])
    meta = ctx.attention_work(0, H // KV, 128, None, H, hd)
    k = torch.randn(pages, KV, P, hd, device=DEV).to(torch.bfloat16)
    v = torch.randn(pages, KV, P, hd, device=DEV).to(torch.bfloat16)
    qkv = torch.randn(B, (H + 2 * KV) * hd, device=DEV).to(torch.bfloat16)
    bias = torch.randn((H + 2 * KV) * hd, device=DEV)
    inv_freq = (1e6 ** (-torch.arange(0, hd, 2, dtype=torch.float32) / hd)).to(DEV)
    out = torch.empty(B, H * hd, dtype=torch.bfloat16, device=DEV)
    splits = ops.fused_decode_splits(B, KV, ctx_len + 1, torch.device(DEV))
    run = lambda: ops.attention_decode_fused(qkv, bias, k, v, out, meta, ctx.positions, ctx.group(0).slots, inv_freq,
                                             B, H, KV, hd, hd ** -0.5, None, P, splits=splits)
    return run, B * (ctx_len + 1) * KV * hd * 2 * 2, splits


def main():
    what = sys.argv[1] if len(sys.argv) > 1 else "all"
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)
    if what in ("skinny", "all"):
        for name, N, K, sw in (("qkv", 4608, 3584, False), ("gate_up", 37888, 3584, True), ("down", 3584, 18944, False)):
            w = (torch.randn(N, K, device=DEV) * 0.02).to(torch.bfloat16)
            x = torch.randn(8, K, device=DEV).to(torch.bfloat16)
            t = timed(lambda: ops.gemm_skinny(x, w, None, torch.bfloat16, swiglu=sw), flush)
            print(f"gemm_skinny {name} M=8: {t * 1e3:.1f} us, {N * K * 2 / t / 1e6:.0f} GB/s")
            for M in (1, 8, 16):        # the library GEMM and the kernel side by side, plain epilogue
                xm = torch.randn(M, K, device=DEV).to(torch.bfloat16)
                tl = timed(lambda: torch.mm(xm, w.t()), flush)
                ts = timed(lambda: ops.gemm_skinny(xm, w, None, torch.bfloat16), flush)
                print(f"  {name} M={M}: library {tl * 1e3:.1f} us ({N * K * 2 / tl / 1e6:.0f} GB/s), "
                      f"gemm_skinny {ts * 1e3:.1f} us ({N * K * 2 / ts / 1e6:.0f} GB/s)")
    if what in ("sgemm", "all"):
        # the float32 path's own GEMM: few rows stream the weights (GB/s), many rows multiply (TFLOP/s)
        for name, N, K in (("qkv", 4608, 3584), ("o", 3584, 3584), ("gate_up", 37888, 3584), ("down", 3584, 18944)):
            w = torch.randn(N, K, device=DEV) * 0.02
            for M in (1, 8, 16, 64, 2048):
                if M == 2048 and name == "o":
                    continue
                x = torch.randn(M, K, device=DEV)
                out = torch.empty(M, N, device=DEV)
                t = timed(lambda: ops.sgemm_nt(x, w, None, out), flush, n=3)
                print(f"sgemm {name} M={M}: {t * 1e3:.1f} us, {N * K * 4 / t / 1e6:.0f} GB/s of weights, "
                      f"{2 * M * N * K / t / 1e9:.1f} TFLOP/s")
            del w
    if what == "sgemm_small":
        # one launch each of the float32 kernels on a case small enough for a full ncu capture
        # (the weights, 136 MB, still exceed the L2)
        w = torch.randn(9472, 3584, device=DEV) * 0.02
        for M in (8, 16, 512):
            x = torch.randn(M, 3584, device=DEV)
            out = torch.empty(M, 9472, device=DEV)
            t = timed(lambda: ops.sgemm_nt(x, w, None, out), flush, n=3)
            print(f"sgemm N=9472 K=3584 M={M}: {t * 1e3:.1f} us, {9472 * 3584 * 4 / t / 1e6:.0f} GB/s of weights, "
                  f"{2 * M * 9472 * 3584 / t / 1e9:.1f} TFLOP/s")
    if what in ("attn_decode", "all"):
        for B in (8, 64):
            run, kv_bytes = attention_case([(2047, 1)] * B)
            t = timed(run, flush)
            print(f"attention decode B={B} ctx 2048: {t * 1e3:.1f} us, {kv_bytes / t / 1e6:.0f} GB/s")
    if what in ("attn_f32", "all"):
        # the float32 path's attention: decoded tokens of 8 requests, and a prompt of 2,048 tokens
        run, kv_bytes = attention_case([(2047, 1)] * 8, kind="simple", dtype=torch.float32)
        t = timed(run, flush)
        print(f"float32 attention decode B=8 ctx 2048: {t * 1e3:.1f} us, {kv_bytes / t / 1e6:.0f} GB/s")
        run, _ = attention_case([(0, 2048)], kind="simple", dtype=torch.float32)
        t = timed(run, flush, n=3)
        print(f"float32 attention prefill 2048 tokens: {t * 1e3:.1f} us, "
              f"{2 * 2 * 28 * 128 * (2048 * 2049 // 2) / t / 1e9:.1f} TFLOP/s")
    if what in ("attn_fused", "all"):
        for B, ctx_len in ((1, 2048), (8, 2048), (8, 8192), (64, 2048)):
            run, kv_bytes, splits = fused_decode_case(B, ctx_len)
            t = timed(run, flush)
            print(f"fused decode attention B={B} ctx {ctx_len} ({splits} blocks a cluster): {t * 1e3:.1f} us, "
                  f"{kv_bytes / t / 1e6:.0f} GB/s")
    if what in ("attn_prefill", "all"):
        for kind in ("mma", "tc5"):
            for T in (2048, 8192):
                run, _ = attention_case([(0, T)], kind=kind)
                t = timed(run, flush)
                flops = 2 * 2 * 28 * 128 * (T * (T + 1) // 2)
                print(f"attention prefill {T} tokens ({kind}): {t * 1e3:.1f} us, {flops / t / 1e9:.0f} TFLOP/s")
    if what in ("tc5", "all"):
        w = (torch.randn(37888, 3584, device=DEV) * 0.02).to(torch.bfloat16)
        x = torch.randn(2048, 3584, device=DEV).to(torch.bfloat16)
        t = timed(lambda: ops.gemm_tc5(x, w, torch.bfloat16, swiglu=True), flush)
        print(f"gemm_tc5 gate_up+SwiGLU M=2048: {t * 1e3:.1f} us, {2 * 2048 * 37888 * 3584 / t / 1e9:.0f} TFLOP/s")
        t = timed(lambda: torch.mm(x, w.t()), flush)
        print(f"library GEMM gate_up M=2048: {t * 1e3:.1f} us, {2 * 2048 * 37888 * 3584 / t / 1e9:.0f} TFLOP/s")
        del w, x
    if what in ("stream", "all"):
        # gemm_stream (tcgen05, weights as the streamed operand) beside the library GEMM (followed by
        # silu_mul for gate/up) and gemm_skinny, decode shapes of the 7B model, 8 to 64 rows
        for name, N, K, sw in (("qkv", 4608, 3584, False), ("o", 3584, 3584, False), ("gate_up", 37888, 3584, True),
                               ("down", 3584, 18944, False)):
            w = (torch.randn(N, K, device=DEV) * 0.02).to(torch.bfloat16)
            for M in (8, 16, 32, 64):
                x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
                t = timed(lambda: ops.gemm_stream(x, w, torch.bfloat16, swiglu=sw), flush)
                if sw:
                    act = torch.empty(M, N // 2, dtype=torch.bfloat16, device=DEV)
                    tl = timed(lambda: ops.silu_mul(torch.mm(x, w.t()), act), flush)
                else:
                    tl = timed(lambda: torch.mm(x, w.t()), flush)
                row = f"gemm_stream {name} M={M}: {t * 1e3:.1f} us ({N * K * 2 / t / 1e6:.0f} GB/s); " \
                      f"library{' + silu_mul' if sw else ''} {tl * 1e3:.1f} us"
                if M <= 16:
                    ts = timed(lambda: ops.gemm_skinny(x, w, None, torch.bfloat16, swiglu=sw), flush)
                    row += f"; gemm_skinny {ts * 1e3:.1f} us"
                print(row)
            del w
    if what == "tc5_shapes":
        # gemm_tc5 beside the library over the prompt shapes of the 7B model; the fused SwiGLU
        # epilogue against the library GEMM followed by the silu_mul kernel
        for M in (256, 512, 1024, 2048, 4096, 8192):
            for name, N, K, sw in (("qkv", 4608, 3584, False), ("o", 3584, 3584, False),
                                   ("gate_up", 37888, 3584, True), ("down", 3584, 18944, False)):
                w = (torch.randn(N, K, device=DEV) * 0.02).to(torch.bfloat16)
                x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
                t = timed(lambda: ops.gemm_tc5(x, w, torch.bfloat16, swiglu=sw), flush)
                if sw:
                    act = torch.empty(M, N // 2, dtype=torch.bfloat16, device=DEV)
                    tl = timed(lambda: ops.silu_mul(torch.mm(x, w.t()), act), flush)
                else:
                    tl = timed(lambda: torch.mm(x, w.t()), flush)
                print(f"M={M} {name}: gemm_tc5 {t * 1e3:.1f} us, {2 * M * N * K / t / 1e9:.0f} TFLOP/s; "
                      f"library{' + silu_mul' if sw else ''} {tl * 1e3:.1f} us")
                del w
    if what in ("sample", "all"):
        V = 152064
        for B in (1, 8, 64, 256):
            logits = torch.randn(B, V, device=DEV) * 3
            u = torch.rand(B, device=DEV)
            out = torch.empty(B, dtype=torch.int32, device=DEV)
            row = [f"argmax {timed(lambda: ops.argmax(logits, out), flush) * 1e3:.1f} us"]
            for name, (T, k, p) in (("temperature", (0.8, 0, 1.0)), ("+ top-k 50", (0.8, 50, 1.0)), ("+ top-p 0.9", (0.8, 0, 0.9)),
                                    ("+ both", (0.8, 50, 0.9))):
                a = (torch.full((B,), T, device=DEV), torch.full((B,), k, dtype=torch.int32, device=DEV),
                     torch.full((B,), p, device=DEV))
                row.append(f"{name} {timed(lambda: ops.sample(logits, a[0], a[1], a[2], u, out), flush) * 1e3:.1f} us")
            print(f"sampling {B} rows of {V}: " + "; ".join(row))


if __name__ == "__main__":
    main()
