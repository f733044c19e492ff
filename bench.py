#!/usr/bin/env python3
"""Measures decode and prefill of the Qwen2.5-7B-shaped model with random weights on one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 2048]

Prints ONE JSON line.  ``value``: decoded tokens a second at batch 8 from 2,048-token
contexts, timed on the device with CUDA events over K decode steps (each step: one
host-to-device copy of the step's integers, the captured decode graph, the argmax kernel;
no host synchronisation between steps).  ``e2e``: the same through ``Engine.step()``, the
call a user makes: host tokens in, sampled ids read back to the host every step (the engine
launches the next decode step before it reads this one's ids, feeding them on the device),
wall clock between synchronisations.  ``prefill``: one step of a 2,048-token prompt.  ``roofline``: bytes a
decode step has to read (every weight once, and the live requests' keys and values)
divided by its time, against the measured copy bandwidth.  ``points``: decode at batch 1
and 64; decode at batch 8 and 64 from 8,192-token contexts; the float32 path (decode at batch
8, a 2,048-token prompt); and two whole workloads through the scheduler (the Qwen2.5-1.5B
shape with 64 requests of 16 to 2,048 prompt tokens read in portions of 512 and 256 new
tokens each; the Qwen2.5-14B shape with 8 prompts of 8,192 tokens and 512 new tokens each),
each with its fraction of the measured peak where one applies.  Weights (15 GB) are far larger
than L2 and are streamed once per step, so no L2 flush is needed between steps.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIG_7B = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_size=3584,
                 num_hidden_layers=28, num_attention_heads=28, num_key_value_heads=4,
                 intermediate_size=18944, vocab_size=152064, rope_theta=1000000.0, rms_norm_eps=1e-6,
                 tie_word_embeddings=False, max_position_embeddings=32768, use_sliding_window=False,
                 hidden_act="silu", eos_token_id=151645)
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = dict(FALLBACK_PEAKS, source="fallback")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            if "hbm_gbs" in d:
                out["hbm_gbs"] = float(d["hbm_gbs"])
            if "bf16_tflops" in d:
                out["bf16_tflops"] = float(d["bf16_tflops"])
            if "bf16_tflops_sustained" in d:
                out["bf16_tflops_sustained"] = float(d["bf16_tflops_sustained"])
            out["source"] = "measured"
        except (OSError, ValueError):
            pass
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.samples, self.proc = [], None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        self.active = False

    def _read(self):
        for line in self.proc.stdout:
            if self.active:
                self.samples.append([x.strip() for x in line.split(",")])

    def summary(self):
        if self.proc is not None:
            self.proc.terminate()
        mhz, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                mhz.append(int(float(s[0])))
                mx = max(mx, int(float(s[1])))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(mhz)}


def model_bytes_and_flops(cfg):
    d, L, H, KV = cfg["hidden_size"], cfg["num_hidden_layers"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd, I, V = d // H, cfg["intermediate_size"], cfg["vocab_size"]
    per_layer = (H + 2 * KV) * hd * d + d * H * hd + 2 * I * d + d * I
    small = (H + 2 * KV) * hd + 2 * d
    weight_bytes = 2 * (L * per_layer + V * d) + 4 * (L * small + d)   # matrices bf16, vectors float32
    kv_bytes_per_token = L * 2 * KV * hd * 2
    linear_flops_per_token = 2 * L * per_layer
    return weight_bytes, kv_bytes_per_token, linear_flops_per_token, (L, H, hd, V, d)


def prepare_decode(engine, batch, context, new_tokens, seed):
    """Submits ``batch`` random prompts of ``context`` tokens and runs steps until every
    request is decoding."""
    import torch
    from paged_batch_engine_b200 import SamplingParams
    g = torch.Generator().manual_seed(seed)
    vocab = engine.runner.model.spec.vocab_size
    reqs = [engine.add_request(torch.randint(0, vocab, (context,), generator=g).tolist(),
                               SamplingParams(max_new_tokens=new_tokens, ignore_eos=True))
            for _ in range(batch)]
    while any(not r.is_decode for r in reqs):
        engine.step()
        engine.drain()
    return reqs


def time_decode_device(engine, reqs, steps, warmup):
    """K decode steps back to back on the device: integers in, graph, argmax; no host sync."""
    import torch
    from paged_batch_engine_b200.csrc import ops
    from paged_batch_engine_b200.engine.batch import StepEntry
    runner, cache = engine.runner, engine.runner.cache
    g = torch.Generator().manual_seed(1)
    vocab = runner.model.spec.vocab_size
    feed = torch.randint(0, vocab, (steps + warmup, len(reqs)), generator=g).tolist()
    out_ids = torch.empty(len(reqs), dtype=torch.int32, device=runner.device)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = 0

    def one(i):
        entries = [StepEntry(r.handle, [feed[i][j]], [0]) for j, r in enumerate(reqs)]
        for e in entries:
            if not cache.reserve(e.handle, 1):
                raise RuntimeError("the bench's cache pool is too small")
        logits = runner.step(entries, commit=True, decode_graph=True)
        ops.argmax(logits, out_ids)
    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    launches0 = ops.launch_count()
    replays0 = runner.graphs.replays
    start.record()
    for i in range(warmup, warmup + steps):
        one(i)
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop)
    own = (ops.launch_count() - launches0) + (runner.graphs.replays - replays0) * runner.graphs.launches_per_replay
    for r in reqs:      # keep the scheduler's view in step with the cache
        r.computed = cache.context_len(r.handle)
        r.outputs = r.outputs + [0] * (r.computed + 1 - len(r.prompt) - len(r.outputs))
    return ms / steps, own


def time_decode_e2e(engine, steps, warmup):
    import torch
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        engine.step()
    torch.cuda.synchronize()
    ms = (time.perf_counter() - t0) * 1e3 / steps
    engine.drain()
    return ms


def finish(engine, reqs):
    for r in reqs:
        engine.scheduler.cancel(r)
    engine.scheduler.pop_finished()


def time_prefill(engine, tokens, repeats, seed=5):
    import torch
    from paged_batch_engine_b200.engine.batch import StepEntry
    runner, cache = engine.runner, engine.runner.cache
    g = torch.Generator().manual_seed(seed)
    vocab = runner.model.spec.vocab_size
    times = []
    for i in range(repeats + 2):
        prompt = torch.randint(0, vocab, (tokens,), generator=g).tolist()
        h = cache.add_request()
        assert cache.reserve(h, tokens)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        runner.step([StepEntry(h, prompt, [tokens - 1])])
        stop.record()
        torch.cuda.synchronize()
        cache.free(h)
        if i >= 2:
            times.append(start.elapsed_time(stop))
    times.sort()
    return times[len(times) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (named in config)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points and the prefill")
    ap.add_argument("--no-extended", action="store_true",
                    help="skip the points at 8,192-token contexts, the float32 path and the scheduler workloads")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a CMake C++/CUDA project without setup.py or pyproject.toml "
                          "(pip: 'not installable') and its build needs glog, armadillo, gtest and re2, "
                          "none of which is in this image"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures a one-GPU engine: --gpus {args.gpus} is not supported (use --gpus 1)")
        return 2
    warmup = max(3, args.warmup)
    steps = max(1, args.steps)

    import torch
    from paged_batch_engine_b200 import Engine
    from paged_batch_engine_b200.config import load_config

    cfg = dict(CONFIG_7B)
    layers_full = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    _, typed = load_config(cfg)
    pk = peaks()
    page = 16
    max_batch = 64 if not args.no_points else args.batch
    # tokens a request may generate: warm-up and timed steps twice (device-timed, then through
    # the entry point) plus what it decodes while the later prompts of its batch are still read
    new_tokens = 2 * (steps + warmup) + 8 + max_batch
    max_len = args.context + new_tokens + 64
    pool_pages = max_batch * ((max_len + page - 1) // page) + 2 * ((2048 + page - 1) // page)
    engine = Engine(typed, dtype=args.dtype, seed=0, page_size=page, num_pages=pool_pages,
                    max_num_seqs=max(max_batch, args.batch), max_num_batched_tokens=4096,
                    prefill_chunk_cap=2048, max_model_len=max_len)
    weight_bytes, kv_per_token, lin_flops, (L, H, hd, V, d) = model_bytes_and_flops(cfg)
    if args.dtype == "float32":
        weight_bytes *= 2
        kv_per_token *= 2

    def decode_point(batch, sampler=None):
        reqs = prepare_decode(engine, batch, args.context, new_tokens, seed=batch)
        if sampler:
            sampler.active = True
        ms_dev, own = time_decode_device(engine, reqs, steps, warmup)
        ms_e2e = time_decode_e2e(engine, steps, warmup)
        if sampler:
            sampler.active = False
        finish(engine, reqs)
        return ms_dev, ms_e2e, own

    sampler = ClockSampler(0)
    ms_dev, ms_e2e, own_launches = decode_point(args.batch, sampler)
    clocks = sampler.summary()
    value = args.batch * 1e3 / ms_dev
    ctx_mid = args.context + warmup + steps / 2
    step_bytes = weight_bytes + args.batch * ctx_mid * kv_per_token
    achieved = step_bytes / (ms_dev * 1e-3) / 1e9
    h2d = engine.runner.graphs.last_h2d_bytes
    result = {
        "metric": "decode tok/s @bs8, Qwen2.5-7B shape, 2048-token contexts", "value": round(value, 2),
        "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": round(ms_dev, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if args.dtype == "bfloat16" else "fp32", "data": "synthetic",
        "config": {"model": "Qwen2.5-7B shape, random weights N(0,0.02)", "global_batch": args.batch,
                   "seq_len": args.context, "parallelism": "single GPU", "layers": cfg["num_hidden_layers"],
                   "layers_full_model": layers_full, "hidden": d, "heads": H,
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": hd,
                   "intermediate": cfg["intermediate_size"], "vocab": V, "kv_page_tokens": page,
                   "context_limit": max_len, "l2": "inputs larger than L2 (weights streamed once per step)",
                   "peaks": pk["source"]},
        "e2e": {"value": round(args.batch * 1e3 / ms_e2e, 2), "unit": "tokens/s", "ms_per_step": round(ms_e2e, 4),
                "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": 4 * args.batch},
        "gpu_launches": int(own_launches),
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "clocks": clocks,
    }
    if not args.no_points:
        points = {}
        for b in (1, 16, 64):
            ms_b, ms_b_e2e, _ = decode_point(b)
            points[f"decode_b{b}"] = round(b * 1e3 / ms_b, 2)
            points[f"decode_b{b}_e2e"] = round(b * 1e3 / ms_b_e2e, 2)
            bytes_b = weight_bytes + b * ctx_mid * kv_per_token
            points[f"decode_b{b}_hbm_frac"] = round(bytes_b / (ms_b * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        result["points"] = points
        T = 2048
        ms_p = time_prefill(engine, T, repeats=5)
        flops = T * lin_flops + 2 * 2 * H * hd * L * (T * (T + 1) // 2) + 2 * V * d
        result["prefill"] = {"value": round(T * 1e3 / ms_p, 1), "tokens": T, "ms": round(ms_p, 3),
                             "frac": round(flops / (ms_p * 1e-3) / 1e12 / pk["bf16_tflops"], 4)}
        if "bf16_tflops_sustained" in pk:
            # the prompt is 25 ms of GEMMs back to back with the clocks at the power cap: the library
            # GEMM's rate in a loop of seconds is the fairer measure beside its burst rate
            result["prefill"]["frac_sustained"] = round(flops / (ms_p * 1e-3) / 1e12 / pk["bf16_tflops_sustained"], 4)
    if not args.no_points and not args.no_extended and args.dtype == "bfloat16" and not args.layers:
        import gc
        points = result["points"]
        del engine
        gc.collect()
        torch.cuda.empty_cache()
        ext_steps = min(steps, 32)
        # (1) long contexts: batch 8 and 64 from 8,192 tokens
        long_ctx = 8192
        new_tokens = 2 * (ext_steps + warmup) + 8 + 64
        max_len = long_ctx + new_tokens + 64
        engine = Engine(typed, dtype="bfloat16", seed=0, page_size=page, num_pages=64 * ((max_len + page - 1) // page) + 8,
                        max_num_seqs=64, max_num_batched_tokens=8192, prefill_chunk_cap=2048, max_model_len=max_len)
        for b in (8, 64):
            reqs = prepare_decode(engine, b, long_ctx, new_tokens, seed=100 + b)
            ms_b, _ = time_decode_device(engine, reqs, ext_steps, warmup)
            finish(engine, reqs)
            bytes_b = weight_bytes + b * (long_ctx + warmup + ext_steps / 2) * kv_per_token
            points[f"decode_b{b}_ctx8192"] = round(b * 1e3 / ms_b, 2)
            points[f"decode_b{b}_ctx8192_hbm_frac"] = round(bytes_b / (ms_b * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        del engine
        gc.collect()
        torch.cuda.empty_cache()
        # (2) the float32 path of the same model: decode at batch 8, a 2,048-token prompt
        f32_steps = min(steps, 16)
        new_tokens = 2 * (f32_steps + warmup) + 16
        max_len = args.context + new_tokens + 64
        engine = Engine(typed, dtype="float32", seed=0, page_size=page,
                        num_pages=8 * ((max_len + page - 1) // page) + 2 * (2048 // page) + 8, max_num_seqs=8,
                        max_num_batched_tokens=4096, prefill_chunk_cap=2048, max_model_len=max_len)
        reqs = prepare_decode(engine, 8, args.context, new_tokens, seed=7)
        ms_b, _ = time_decode_device(engine, reqs, f32_steps, warmup)
        finish(engine, reqs)
        bytes_b = 2 * weight_bytes + 8 * (args.context + warmup + f32_steps / 2) * 2 * kv_per_token
        points["decode_b8_fp32"] = round(8 * 1e3 / ms_b, 2)
        points["decode_b8_fp32_hbm_frac"] = round(bytes_b / (ms_b * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        ms_p = time_prefill(engine, 2048, repeats=1)
        points["prefill_fp32_tok_s"] = round(2048 * 1e3 / ms_p, 1)
        points["prefill_fp32_tflops"] = round(flops / (ms_p * 1e-3) / 1e12, 2)
        del engine
        gc.collect()
        torch.cuda.empty_cache()
        # (3) whole workloads through the scheduler at two further model shapes
        import bench_serving
        for name, key in (("1.5b", "serve_1p5b_64req"), ("14b", "serve_14b_8x8192")):
            # one untimed round first, as the reference's benchmark app runs with --warmup-rounds=1;
            # that round's own rate (every decode graph captured inside it) is kept beside it
            line = bench_serving.run_workload(name, warmup_rounds=1)
            points[f"{key}_tok_s"] = line["value"]
            points[f"{key}_first_round_tok_s"] = line["first_round_value"]
            points[f"{key}_wall_s"] = line["wall_s"]
            points[f"{key}_ttft_p50_ms"] = line["ttft_p50_ms"]
            points[f"{key}_gap_p50_ms"] = line["token_gap_p50_ms"]
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
