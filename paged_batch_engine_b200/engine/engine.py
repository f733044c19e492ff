"""The Python entry point: a model folder (or a configuration with random weights) to
generated tokens on one GPU.

    engine = Engine("path/to/model", dtype="bfloat16")
    results = engine.generate([[1, 2, 3], [4, 5]], SamplingParams(max_new_tokens=32))

``generate`` submits the prompts to the scheduler and loops ``step()`` until all are done:
schedule -> build the batch -> run the step function -> sample on the device -> read the
sampled ids back -> update the requests.  This is the loop of the reference's offline app
(infMain/source/serving/serving_benchmark_app.cpp:742-838) with the model's
``forward_mixed_batch`` and ``batch_sample`` behind it.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Union

import torch

from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .batch import StepEntry
from .metrics import final_summary, nvtx_range
from .runner import ModelRunner, _parse_dtype
from .scheduler import Request, Scheduler, SchedulerConfig, SchedulerOutput


@dataclass
class GenerationResult:
    request_id: int
    prompt_tokens: List[int]
    output_tokens: List[int]
    finish_reason: str
    preemptions: int = 0
    request: Optional[Request] = None      # the scheduler's record (times, counters) behind this result


class Engine:
    def __init__(self, model: Union[str, object], dtype="bfloat16", device="cuda:0", seed: int = 0,
                 page_size: int = 16, num_pages: Optional[int] = None,
                 kv_cache_memory_utilization: float = 0.80, max_num_seqs: int = 256,
                 max_num_batched_tokens: int = 2048, prefill_chunk_cap: int = 512,
                 long_prefill_token_threshold: int = 0, max_model_len: Optional[int] = None,
                 use_cuda_graphs: bool = True, decode_ahead: bool = True):
        """``model``: a folder with config.json and safetensors, or a typed configuration /
        config dict, in which case the weights are random from ``seed``.  ``num_pages``:
        pages per layer group; if None the cache takes ``kv_cache_memory_utilization`` of the
        free device memory minus a reserve, as the reference plans its pool
        (infMain/source/model/serving_memory_planner.cpp:41-106)."""
        self.dtype = _parse_dtype(dtype)
        self.device = torch.device(device)
        kw = dict(page_tokens=page_size, max_requests=max(max_num_seqs, 1), max_context=max_model_len)
        if isinstance(model, str):
            build = lambda **k: ModelRunner.from_folder(model, dtype=self.dtype, device=device, **k)
        else:
            build = lambda **k: ModelRunner.from_random(model, seed=seed, dtype=self.dtype, device=device, **k)
        if num_pages is None:
            # load the weights first with a one-page pool, then size the pool from what is free
            probe = build(num_pages=1, **kw)
            per_page = probe.storage.bytes_per_token() * page_size
            free, _total = torch.cuda.mem_get_info(self.device)
            util = min(0.95, max(0.01, kv_cache_memory_utilization))
            reserve = max(256 << 20, int(0.05 * free))
            num_pages = max(1, int((free * util - reserve) // max(per_page, 1)))
            if max_model_len:
                num_pages = min(num_pages, max_num_seqs * ((max_model_len + page_size - 1) // page_size))
            self.runner = ModelRunner(probe.model, num_pages=num_pages, **kw)
            del probe
        else:
            self.runner = build(num_pages=num_pages, **kw)
        spec = self.runner.model.spec
        self.max_model_len = int(max_model_len or spec.max_position)
        self.scheduler = Scheduler(
            SchedulerConfig(max_num_seqs=max_num_seqs, max_num_batched_tokens=max_num_batched_tokens,
                            prefill_chunk_cap=prefill_chunk_cap,
                            long_prefill_token_threshold=long_prefill_token_threshold,
                            max_model_len=self.max_model_len),
            self.runner.cache, spec.eos_token_ids)
        self.sampler = Sampler(self.device, max_requests=max_num_seqs)
        self.use_cuda_graphs = use_cuda_graphs
        self.decode_ahead = bool(decode_ahead and use_cuda_graphs)   # pipeline decode steps one deep
        self._pending = None
        self.profile = dict(schedule=0.0, forward=0.0, sample=0.0, process=0.0, steps=0)

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None) -> Request:
        vocab = self.runner.model.spec.vocab_size
        for t in prompt:
            if not (0 <= int(t) < vocab):
                raise ValueError(f"token id {t} is outside the vocabulary of {vocab}")
        if len(prompt) >= self.max_model_len:
            raise ValueError(f"a prompt of {len(prompt)} tokens leaves no room under max_model_len "
                             f"{self.max_model_len}")
        return self.scheduler.add_request(prompt, params)

    def has_unfinished_requests(self) -> bool:
        return self._pending is not None or self.scheduler.has_active_requests()

    # ------------------------------------------------------------------ one step
    def step(self) -> List[Request]:
        """Runs one scheduler step; returns the requests known to have finished.

        Steps of decoded tokens only are pipelined one deep (``decode_ahead``): such a step is
        launched and left running; the next call first schedules and launches the step after
        it - its token ids stay on the device, where the running step's sampler leaves them -
        and only then reads the running step's tokens and does its bookkeeping, so the host's
        work hides behind the device's.  A request's tokens therefore become known one call
        later than they are computed; ``drain()`` brings the host up to date."""
        with nvtx_range("engine.step"):
            return self._step()

    def _step(self) -> List[Request]:
        t0 = time.perf_counter()
        if self._pending is not None:
            prev, self._pending = self._pending, None
            ahead = self.scheduler.schedule_ahead(prev[0]) if self.decode_ahead else None
            if ahead is not None:
                t1 = time.perf_counter()
                self._pending = self._launch(ahead, prev[1])
                self.profile["schedule"] += t1 - t0
                self.profile["forward"] += time.perf_counter() - t1
                self._finish(prev)               # adds its own wait and bookkeeping to the profile
                self.profile["steps"] += 1
                return self._pop_finished()
            self._finish(prev)
            t0 = time.perf_counter()
        with nvtx_range("schedule"):
            out = self.scheduler.schedule_step()
        t1 = time.perf_counter()
        self.profile["schedule"] += t1 - t0
        self.profile["steps"] += 1
        if out.entries:
            launched = self._launch(out, None)
            t2 = time.perf_counter()
            self.profile["forward"] += t2 - t1
            if launched[3] is not None and self.decode_ahead:
                self._pending = launched            # read by the next call, behind the next launch
            else:
                self._finish(launched)
                self.profile["sample"] += time.perf_counter() - t2
        return self._pop_finished()

    def _pop_finished(self) -> List[Request]:
        done = self.scheduler.pop_finished()
        for r in done:
            self.sampler.untrack(r.request_id)
        return done

    def drain(self) -> List[Request]:
        """Waits for a step left running by ``step()`` and does its bookkeeping."""
        if self._pending is not None:
            prev, self._pending = self._pending, None
            self._finish(prev)
        return self._pop_finished()

    def _launch(self, out, device_tokens):
        """Enqueues the step and its sampling.  Returns (out, ids on the device, ids in pinned
        host memory, event) for a step whose ids are read later, (out, None, ids, None) for one
        whose ids are already on the host."""
        entries = [StepEntry(e.request.handle, e.tokens, [len(e.tokens) - 1] if e.samples else [])
                   for e in out.entries]
        rows = [e for e in out.entries if e.samples]
        decode_only = self.use_cuda_graphs and len(rows) == len(entries) and all(len(e.tokens) == 1 for e in rows)
        with nvtx_range("forward"):
            logits = self.runner.step(entries, commit=False, decode_graph=decode_only, device_tokens=device_tokens)
        params = [e.request.params for e in rows]
        counters = [e.request.sampling_counter if e.counter is None else e.counter for e in rows]
        later = decode_only and self.decode_ahead and self.runner.graphs is not None and \
            self.runner.graphs.eligible(entries)
        if device_tokens is not None and not later:
            raise RuntimeError("a step scheduled ahead must be a captured decode step")
        # a request with a repetition penalty gets its row of seen tokens on the device the first
        # time it is sampled (all it has so far: after a preemption its generated tokens too)
        keys = [e.request.request_id for e in rows]
        vocab = self.runner.model.spec.vocab_size
        for e in rows:
            if e.request.params.repetition_penalty != 1.0 and not self.sampler.tracked(e.request.request_id):
                self.sampler.track(e.request.request_id, e.request.tokens, vocab)
        if later:
            with nvtx_range("sample"):
                dev, host, event = self.sampler.sample_async(logits, params, counters, keys)
            return out, dev, host, event
        if rows:
            with nvtx_range("sample"):
                ids = self.sampler.sample(logits, params, counters, keys=keys)
        else:
            from ..csrc import ops
            ops.raise_on_kernel_status(self.device)      # synchronises
            ids = []
        return out, None, ids, None

    def _finish(self, launched) -> None:
        out, _dev, ids, event = launched
        t0 = time.perf_counter()
        if event is not None:
            ids = self.sampler.read_async(ids, event)     # raises if a kernel's bounded wait ran out
        t1 = time.perf_counter()
        with nvtx_range("process_outputs"):
            self.scheduler.process_outputs(out, ids)
        self.profile["sample"] += t1 - t0
        self.profile["process"] += time.perf_counter() - t1

    # ------------------------------------------------------------------ whole requests
    def generate(self, prompts: Sequence[Sequence[int]],
                 sampling_params: Union[SamplingParams, Sequence[SamplingParams], None] = None
                 ) -> List[GenerationResult]:
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params or SamplingParams()] * len(prompts)
        if len(sampling_params) != len(prompts):
            raise ValueError("one SamplingParams per prompt, or one for all")
        reqs = [self.add_request(p, sp) for p, sp in zip(prompts, sampling_params)]
        finished: Dict[int, Request] = {r.request_id: r for r in self._pop_finished()}
        while self.has_unfinished_requests():
            for r in self.step():
                finished[r.request_id] = r
        for r in self.drain():
            finished[r.request_id] = r
        return [GenerationResult(r.request_id, list(r.prompt), list(r.outputs), r.finish_reason,
                                 r.preemptions, r) for r in reqs]

    def summary(self, requests, wall_s: float) -> Dict[str, float]:
        """The run's FINAL_SUMMARY record (see ``engine.metrics``) for these requests."""
        return final_summary(requests, self.scheduler.metrics, self.profile, wall_s)


def generate(model, prompts, sampling_params=None, **engine_args) -> List[List[int]]:
    """One call: build an engine for ``model`` and return the generated token ids."""
    eng = Engine(model, **engine_args)
    return [r.output_tokens for r in eng.generate(prompts, sampling_params)]
