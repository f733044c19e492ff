"""Per-request and whole-run records in the reference's own words, and optional NVTX ranges.

The reference's offline app prints one ``REQUEST_METRIC`` line per request (time to first
token, mean gap between tokens, latency, finish reason) and one ``FINAL_SUMMARY`` line
(infMain/source/serving/serving_benchmark_app.cpp:212-224, 318-391), with the times
defined in infMain/include/serving/sequence_state.h:140-165: time to first token from
arrival to the first sampled token, the mean token gap (first token to last token over
tokens - 1), latency from arrival to the end.  The same key=value lines are made here from
the scheduler's requests and counters; keys of subsystems this engine does not have (radix
cache, host tier, priorities) are left out.

NVTX ranges (infMain/include/base/nvtx_utils.h:34-95 wraps steps, schedule, forward, layers,
sampling and output processing) are pushed only when PBE_NVTX=1 is in the environment, so
that a run without a profiler pays nothing.
"""
from __future__ import annotations

import contextlib
import os
from typing import Dict, Iterable, List, Sequence


def nvtx_enabled() -> bool:
    return os.environ.get("PBE_NVTX", "0") == "1"


@contextlib.contextmanager
def _pushed(name: str):
    import torch
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


_NULL = contextlib.nullcontext()


def nvtx_range(name: str):
    """``with nvtx_range("forward"):`` - a named range for a profiler's timeline when PBE_NVTX=1,
    nothing otherwise."""
    return _pushed(name) if nvtx_enabled() else _NULL


def _ms(a, b) -> float:
    return 0.0 if a is None or b is None else (b - a) * 1e3


def ttft_ms(req) -> float:
    return _ms(req.arrival_time, req.first_token_time)


def itl_ms(req) -> float:
    """Mean gap between the request's tokens (0 for fewer than two)."""
    if req.generated <= 1 or req.first_token_time is None:
        return 0.0
    return _ms(req.first_token_time, req.last_token_time) / (req.generated - 1)


def latency_ms(req) -> float:
    return _ms(req.arrival_time, req.finished_time)


def request_metric_line(req) -> str:
    return ("REQUEST_METRIC"
            f" client_request_id={req.request_id}"
            f" status={'failed' if req.status == 'failed' else 'ok'}"
            f" prompt_tokens={len(req.prompt)}"
            f" generated_tokens={req.generated}"
            f" output_tokens={len(req.outputs)}"
            f" ttft_ms={ttft_ms(req):.3f}"
            f" itl_ms={itl_ms(req):.3f}"
            f" latency_ms={latency_ms(req):.3f}"
            f" finish_reason={req.finish_reason or 'completed'}"
            f" preemptions={req.preemptions}")


def percentile(values: Sequence[float], q: float) -> float:
    if not values:
        return 0.0
    v = sorted(values)
    pos = q * (len(v) - 1)
    lo = int(pos)
    hi = min(lo + 1, len(v) - 1)
    return v[lo] + (v[hi] - v[lo]) * (pos - lo)


def _mean(values: Sequence[float]) -> float:
    return sum(values) / len(values) if values else 0.0


def final_summary(requests: Iterable, scheduler_metrics: Dict[str, int], profile: Dict[str, float],
                  wall_s: float) -> Dict[str, float]:
    """The whole run as a dictionary, keys as in the reference's FINAL_SUMMARY."""
    reqs: List = list(requests)
    ok = [r for r in reqs if r.status != "failed"]
    gaps: List[float] = []
    for r in ok:
        t = r.token_times
        gaps += [(b - a) * 1e3 for a, b in zip(t, t[1:])]
    ttft = [ttft_ms(r) for r in ok if r.first_token_time is not None]
    itl = [itl_ms(r) for r in ok if r.generated > 1]
    lat = [latency_ms(r) for r in reqs if r.finished_time is not None]
    steps = max(1, int(profile.get("steps", 0)))
    m = scheduler_metrics
    generated = sum(r.generated for r in reqs)
    out = {
        "total_steps": m.get("steps", 0),
        "active_steps": m.get("steps", 0) - m.get("no_progress_steps", 0),
        "decode_only_steps": m.get("decode_only_steps", 0),
        "completed_requests": len(ok),
        "failed_requests": len(reqs) - len(ok),
        "total_decode_tokens": m.get("decode_tokens", 0),
        "total_prefill_tokens": m.get("prefill_tokens", 0),
        "total_batched_tokens": m.get("decode_tokens", 0) + m.get("prefill_tokens", 0),
        "scheduler_no_progress_steps": m.get("no_progress_steps", 0),
        "scheduler_preemptions": m.get("preemptions", 0),
        "scheduler_ahead_steps": m.get("ahead_steps", 0),
        "scheduler_dropped_tokens": m.get("dropped_tokens", 0),
        "max_waiting_queue": m.get("max_waiting_queue", 0),
        "max_running_queue": m.get("max_running_queue", 0),
        "wall_ms": wall_s * 1e3,
        "throughput_tps": generated / wall_s if wall_s > 0 else 0.0,
        "avg_schedule_ms": 1e3 * profile.get("schedule", 0.0) / steps,
        "avg_forward_ms": 1e3 * profile.get("forward", 0.0) / steps,
        "avg_sample_ms": 1e3 * profile.get("sample", 0.0) / steps,
        "avg_process_outputs_ms": 1e3 * profile.get("process", 0.0) / steps,
        "avg_step_ms": wall_s * 1e3 / steps,
        "ttft_ms": _mean(ttft), "ttft_p50_ms": percentile(ttft, 0.5), "ttft_p95_ms": percentile(ttft, 0.95),
        "ttft_p99_ms": percentile(ttft, 0.99),
        "token_gap_count": len(gaps), "token_gap_p50_ms": percentile(gaps, 0.5),
        "token_gap_p95_ms": percentile(gaps, 0.95), "token_gap_p99_ms": percentile(gaps, 0.99),
        "itl_ms": _mean(itl), "itl_p50_ms": percentile(itl, 0.5), "itl_p95_ms": percentile(itl, 0.95),
        "itl_p99_ms": percentile(itl, 0.99),
        "latency_ms": _mean(lat), "latency_p50_ms": percentile(lat, 0.5), "latency_p95_ms": percentile(lat, 0.95),
        "latency_p99_ms": percentile(lat, 0.99),
    }
    return out


def final_summary_line(summary: Dict[str, float]) -> str:
    def fmt(v):
        return f"{v:.3f}" if isinstance(v, float) else str(v)
    return "FINAL_SUMMARY " + " ".join(f"{k}={fmt(v)}" for k, v in summary.items())
