#!/usr/bin/env python3
"""Whole workloads through the scheduler and the Python entry point, with random weights.

    python bench_serving.py [--workload 1.5b|14b|7b] [--requests N] [--layers L]

``1.5b``: the Qwen2.5-1.5B shape, 64 requests whose prompt lengths are uniform in 16..2048
(seeded), prompts read in portions of 512 beside the decoding requests, 256 new tokens each.
``14b``: the Qwen2.5-14B shape, 8 prompts of 8,192 tokens, then 512 new tokens each.
``7b``: the Qwen2.5-7B shape under the 1.5b workload.
``prompt-sweep``: one prompt of 128 .. 32,768 tokens, whole or in portions, through the model
runner (8 layers of the 7B shape unless --layers says otherwise).

Everything goes through ``Engine.generate``: admission, portions under the token budget,
mixed steps of prompt portions beside decoded tokens, sampling (greedy), finishing.  Prints
ONE JSON line: generated tokens a second over the wall clock of the whole run, the prompt
tokens a second, the number of steps and the host's share of the time by phase (schedule,
forward = enqueueing the step, sample = waiting for the device and reading the ids, process).
It is a workload check beside ``bench.py``, whose line is the headline.
"""
import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def shape(hidden, layers, heads, kv, inter, vocab, tied):
    return dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_size=hidden,
                num_hidden_layers=layers, num_attention_heads=heads, num_key_value_heads=kv,
                intermediate_size=inter, vocab_size=vocab, rope_theta=1000000.0, rms_norm_eps=1e-6,
                tie_word_embeddings=tied, max_position_embeddings=32768, use_sliding_window=False,
                hidden_act="silu", eos_token_id=151645)


SHAPES = {
    "1.5b": shape(1536, 28, 12, 2, 8960, 151936, True),
    "7b": shape(3584, 28, 28, 4, 18944, 152064, False),
    "14b": shape(5120, 48, 40, 8, 13824, 152064, False),
}


def prompt_sweep(layers):
    """One prompt of several lengths, whole or in portions, through ``ModelRunner.step`` (the
    Qwen2.5-7B shape with ``layers`` layers); CUDA-event time of the whole prompt, median of 3."""
    import torch
    from paged_batch_engine_b200 import Engine
    from paged_batch_engine_b200.config import load_config
    from paged_batch_engine_b200.engine.batch import StepEntry
    cfg = dict(SHAPES["7b"])
    layers_full = cfg["num_hidden_layers"]
    cfg["num_hidden_layers"] = layers or 8
    _, typed = load_config(cfg)
    eng = Engine(typed, dtype="bfloat16", seed=0, page_size=16, num_pages=2200, max_num_seqs=4,
                 max_num_batched_tokens=40000, prefill_chunk_cap=40000, max_model_len=34000)
    runner, cache = eng.runner, eng.runner.cache
    g = torch.Generator().manual_seed(0)
    d, L, H, KV = cfg["hidden_size"], cfg["num_hidden_layers"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd, inter = d // H, cfg["intermediate_size"]
    lin = 2 * L * ((H + 2 * KV) * hd * d + d * H * hd + 3 * inter * d)
    rows = []
    for total, chunk in ((128, 128), (512, 512), (2048, 2048), (2048, 512), (8192, 8192), (8192, 2048),
                         (8192, 512), (32768, 8192), (32768, 2048)):
        times = []
        for _ in range(3):
            prompt = torch.randint(0, 1000, (total,), generator=g).tolist()
            h = cache.add_request()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            for lo in range(0, total, chunk):
                n = min(chunk, total - lo)
                assert cache.reserve(h, n)
                runner.step([StepEntry(h, prompt[lo:lo + n], [n - 1] if lo + n == total else [])])
            stop.record()
            torch.cuda.synchronize()
            cache.free(h)
            times.append(start.elapsed_time(stop))
        ms = sorted(times)[1]
        flops = lin * total + 2 * 2 * H * hd * L * (total * (total + 1) // 2)
        rows.append({"tokens": total, "portion": chunk, "ms": round(ms, 2), "tok_per_s": round(total / ms * 1e3),
                     "tflops": round(flops / ms / 1e9)})
    print(json.dumps({"metric": "prompt tok/s over prompt lengths and portion sizes, Qwen2.5-7B shape",
                      "layers": L, "layers_full_model": layers_full, "dtype": "bf16", "rows": rows}))


def run_workload(workload, requests=0, new_tokens=0, layers=0, max_batched_tokens=0, prefill_chunk=0,
                 warmup_rounds=0):
    """One whole workload through ``Engine.generate``; returns its record (a dict).
    ``warmup_rounds``: untimed runs of the whole workload before the timed one, as the reference's
    benchmark app does with --warmup-rounds (serving_benchmark_app.cpp:646-690): the decode graphs
    of every batch size the run meets are then captured before the clock starts."""
    import torch
    from paged_batch_engine_b200 import Engine, SamplingParams
    from paged_batch_engine_b200.config import load_config
    from paged_batch_engine_b200.csrc import ops

    cfg = dict(SHAPES[workload])
    layers_full = cfg["num_hidden_layers"]
    if layers:
        cfg["num_hidden_layers"] = layers
    _, typed = load_config(cfg)
    g = torch.Generator().manual_seed(2024)
    if workload == "14b":
        n = requests or 8
        lengths = [8192] * n
        new_tokens = new_tokens or 512
        chunk = prefill_chunk or 2048
    else:
        n = requests or 64
        lengths = torch.randint(16, 2049, (n,), generator=g).tolist()
        new_tokens = new_tokens or 256
        chunk = prefill_chunk or 512
    budget = max_batched_tokens or max(chunk, 2048)
    vocab = cfg["vocab_size"]
    prompts = [torch.randint(0, vocab, (L,), generator=g).tolist() for L in lengths]
    page = 16
    max_len = max(lengths) + new_tokens + 16
    pages = sum((L + new_tokens + page) // page + 1 for L in lengths) + 8
    engine = Engine(typed, dtype="bfloat16", seed=0, page_size=page, num_pages=pages, max_num_seqs=max(n, 1),
                    max_num_batched_tokens=budget, prefill_chunk_cap=chunk, max_model_len=max_len)
    params = SamplingParams(max_new_tokens=new_tokens, ignore_eos=True)
    # warm-up: kernels loaded, graphs captured for the batch sizes of the run's tail
    engine.generate([p[:64] for p in prompts[:min(n, 8)]], SamplingParams(max_new_tokens=4, ignore_eos=True))
    first_round = None
    for _ in range(warmup_rounds):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        done = engine.generate(prompts, params)
        torch.cuda.synchronize()
        if first_round is None:      # the run that meets every batch size for the first time
            first_round = round(sum(len(r.output_tokens) for r in done) / (time.perf_counter() - t0), 1)
    torch.cuda.synchronize()
    for k in engine.profile:
        engine.profile[k] = 0 if k == "steps" else 0.0
    launches0 = ops.launch_count()
    graphs = engine.runner.graphs
    captures0, capture_s0 = len(graphs.graphs), graphs.capture_seconds
    t0 = time.perf_counter()
    results = engine.generate(prompts, params)
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    generated = sum(len(r.output_tokens) for r in results)
    prof = engine.profile
    summary = engine.summary([r.request for r in results], wall)
    line = {
        "metric": f"generated tok/s, Qwen2.5-{workload.upper()} shape, {n} requests through the scheduler",
        "value": round(generated / wall, 1), "unit": "tokens/s", "wall_s": round(wall, 3),
        "first_round_value": first_round, "prompt_tokens": sum(lengths), "prompt_tok_per_s_overall": round(sum(lengths) / wall, 1),
        "generated_tokens": generated, "steps": prof["steps"],
        "host_ms_per_step": {k: round(1e3 * prof[k] / max(prof["steps"], 1), 3)
                             for k in ("schedule", "forward", "sample", "process")},
        "ttft_p50_ms": round(summary["ttft_p50_ms"], 2), "ttft_p95_ms": round(summary["ttft_p95_ms"], 2),
        "token_gap_p50_ms": round(summary["token_gap_p50_ms"], 3), "token_gap_p95_ms": round(summary["token_gap_p95_ms"], 3),
        "preemptions": sum(r.preemptions for r in results),
        "graph_captures": len(graphs.graphs) - captures0,
        "graph_capture_s": round(graphs.capture_seconds - capture_s0, 3),
        "kernel_launches_eager": ops.launch_count() - launches0,
        "config": {"layers": cfg["num_hidden_layers"], "layers_full_model": layers_full, "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "intermediate": cfg["intermediate_size"], "vocab": vocab, "page_tokens": page,
                   "max_batched_tokens": budget, "prefill_chunk": chunk, "new_tokens": new_tokens,
                   "warmup_rounds": warmup_rounds,
                   "dtype": "bf16", "data": "synthetic tokens, random weights"},
    }
    del engine
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="1.5b", choices=sorted(SHAPES) + ["prompt-sweep"])
    ap.add_argument("--requests", type=int, default=0)
    ap.add_argument("--new-tokens", type=int, default=0)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the shape has (named in the line)")
    ap.add_argument("--max-batched-tokens", type=int, default=0)
    ap.add_argument("--prefill-chunk", type=int, default=0)
    ap.add_argument("--warmup-rounds", type=int, default=0,
                    help="untimed runs of the whole workload first (the reference's --warmup-rounds)")
    args = ap.parse_args()
    if args.workload == "prompt-sweep":
        return prompt_sweep(args.layers)
    print(json.dumps(run_workload(args.workload, args.requests, args.new_tokens, args.layers,
                                  args.max_batched_tokens, args.prefill_chunk, args.warmup_rounds)))


if __name__ == "__main__":
    main()
