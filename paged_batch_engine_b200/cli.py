"""Command line in the manner of the reference's demos.

``demo/main_qwen.cpp`` takes a model and generates greedily, then prints ``steps``,
``duration`` and ``steps/s``; ``serving_qwen`` adds ``--key=value`` flags
(infMain/source/serving/serving_config_parser.cpp:133-258).  The flags that concern one
GPU and one model are kept here with their names and meanings; tokenisation is outside
the engine, so prompts are given as token ids.

    pbe-qwen MODEL_DIR --prompt-ids 1,2,3 --prompt-ids 4,5 --max-new-tokens=32
    pbe-qwen --write-random-model DIR --config config.json --seed 0
"""
from __future__ import annotations

import argparse
import json
import sys
import time


def _auto_int(text: str):
    if text == "auto":
        return None
    try:
        v = int(text)
    except ValueError:
        raise argparse.ArgumentTypeError(f"expected an integer or 'auto', got {text!r}")
    if v <= 0:
        raise argparse.ArgumentTypeError("must be positive")
    return v


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="pbe-qwen", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("model", nargs="?", help="folder with config.json and model.safetensors")
    ap.add_argument("--prompt-ids", action="append", default=[], help="comma-separated token ids (repeatable)")
    ap.add_argument("--prompt-file", help="file with one prompt a line: token ids separated by spaces or commas")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--max-new-tokens", type=int, default=256)
    ap.add_argument("--min-new-tokens", type=int, default=0)
    ap.add_argument("--max-batched-tokens", type=_auto_int, default=None, metavar="N|auto")
    ap.add_argument("--prefill-chunk-cap", type=_auto_int, default=None, metavar="N|auto")
    ap.add_argument("--long-prefill-token-threshold", type=int, default=0)
    ap.add_argument("--max-num-seqs", type=int, default=256)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--repetition-penalty", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=0xC0FFEE)
    ap.add_argument("--ignore-eos", action="store_true")
    ap.add_argument("--device-id", type=int, default=0)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--kv-cache-memory-utilization", type=float, default=0.80)
    ap.add_argument("--kv-cache-blocks-per-layer", type=int, default=0, help="pages in the pool; 0: from memory")
    ap.add_argument("--max-model-len", type=int, default=0)
    ap.add_argument("--warmup-rounds", type=int, default=0)
    ap.add_argument("--no-cuda-graphs", action="store_true")
    ap.add_argument("--quiet", action="store_true")
    ap.add_argument("--step-profile", action="store_true")
    ap.add_argument("--request-metrics", action="store_true",
                    help="print a REQUEST_METRIC line per request (time to first token, mean token gap, latency)")
    ap.add_argument("--final-summary", action="store_true",
                    help="print the run's FINAL_SUMMARY line (steps, tokens, scheduler counters, percentiles)")
    ap.add_argument("--write-random-model", metavar="DIR",
                    help="write config.json and model.safetensors with seeded random weights and exit")
    ap.add_argument("--config", help="config.json for --write-random-model")
    ap.add_argument("--weights-seed", type=int, default=0)
    return ap


def _read_prompts(args):
    prompts = []
    for text in args.prompt_ids:
        prompts.append([int(t) for t in text.replace(",", " ").split()])
    if args.prompt_file:
        with open(args.prompt_file) as f:
            for line in f:
                ids = [int(t) for t in line.replace(",", " ").split()]
                if ids:
                    prompts.append(ids)
    return prompts


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if args.write_random_model:
        import torch
        from .config import load_config
        from .engine.runner import build_model
        from .weights import write_random_model
        if not args.config:
            print("--write-random-model needs --config", file=sys.stderr)
            return 2
        _, typed = load_config(args.config)
        model = build_model(typed, torch.float32, "cpu")
        write_random_model(args.write_random_model, typed, model.param_specs(), args.weights_seed,
                           torch.bfloat16 if args.dtype == "bfloat16" else torch.float32)
        print(f"wrote {args.write_random_model}")
        return 0
    if not args.model:
        print("a model folder is required", file=sys.stderr)
        return 2
    prompts = _read_prompts(args)
    if not prompts:
        print("no prompt given (--prompt-ids or --prompt-file)", file=sys.stderr)
        return 2
    from .engine.engine import Engine
    from .sampling.params import SamplingParams
    engine = Engine(args.model, dtype=args.dtype, device=f"cuda:{args.device_id}", page_size=args.page_size,
                    num_pages=args.kv_cache_blocks_per_layer or None,
                    kv_cache_memory_utilization=args.kv_cache_memory_utilization,
                    max_num_seqs=args.max_num_seqs,
                    max_num_batched_tokens=args.max_batched_tokens or 4096,
                    prefill_chunk_cap=args.prefill_chunk_cap or 1024,
                    long_prefill_token_threshold=args.long_prefill_token_threshold,
                    max_model_len=args.max_model_len or None, use_cuda_graphs=not args.no_cuda_graphs)
    params = SamplingParams(max_new_tokens=args.max_new_tokens, min_new_tokens=args.min_new_tokens,
                            ignore_eos=args.ignore_eos, temperature=args.temperature, top_k=args.top_k,
                            top_p=args.top_p, repetition_penalty=args.repetition_penalty, seed=args.seed)
    for _ in range(args.warmup_rounds):
        engine.generate(prompts, params)
    for k in engine.profile:
        engine.profile[k] = 0
    if not args.quiet:
        print("Generating...", flush=True)
    t0 = time.perf_counter()
    results = engine.generate(prompts, params)
    duration = time.perf_counter() - t0
    steps = sum(len(r.output_tokens) for r in results)
    if not args.quiet:
        for r in results:
            print(json.dumps({"request": r.request_id, "prompt_tokens": len(r.prompt_tokens),
                              "output_ids": r.output_tokens, "finish_reason": r.finish_reason}))
    if args.step_profile:
        p = engine.profile
        n = max(1, p["steps"])
        print("STEP_PROFILE " + " ".join(f"{k}_ms={1e3 * p[k] / n:.3f}" for k in
                                          ("schedule", "forward", "sample", "process")) + f" steps={p['steps']}")
    if args.request_metrics or args.final_summary:
        from .engine.metrics import final_summary_line, request_metric_line
        if args.request_metrics:
            for r in results:
                print(request_metric_line(r.request))
        if args.final_summary:
            print(final_summary_line(engine.summary([r.request for r in results], duration)))
    print(f"\nsteps:{steps}")
    print(f"\nduration:{duration:f}")
    print(f"\nsteps/s:{steps / duration if duration > 0 else 0.0:f}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
