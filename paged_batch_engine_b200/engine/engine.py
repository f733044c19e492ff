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
from .runner import ModelRunner, _parse_dtype
from .scheduler import Request, Scheduler, SchedulerConfig, SchedulerOutput


@dataclass
class GenerationResult:
    request_id: int
    prompt_tokens: List[int]
    output_tokens: List[int]
    finish_reason: str
    preemptions: int = 0


class Engine:
    def __init__(self, model: Union[str, object], dtype="bfloat16", device="cuda:0", seed: int = 0,
                 page_size: int = 16, num_pages: Optional[int] = None,
                 kv_cache_memory_utilization: float = 0.80, max_num_seqs: int = 256,
                 max_num_batched_tokens: int = 2048, prefill_chunk_cap: int = 512,
                 long_prefill_token_threshold: int = 0, max_model_len: Optional[int] = None,
                 use_cuda_graphs: bool = True):
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
        self.sampler = Sampler(self.device)
        self.use_cuda_graphs = use_cuda_graphs
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
        return self.scheduler.has_active_requests()

    # ------------------------------------------------------------------ one step
    def step(self) -> List[Request]:
        """Runs one scheduler step; returns the requests that finished in it."""
        t0 = time.perf_counter()
        out = self.scheduler.schedule_step()
        t1 = time.perf_counter()
        sampled: List[int] = []
        if out.entries:
            entries = [StepEntry(e.request.handle, e.tokens, [len(e.tokens) - 1] if e.samples else [])
                       for e in out.entries]
            rows = [e.request for e in out.entries if e.samples]
            decode_only = self.use_cuda_graphs and all(len(e.tokens) == 1 and e.samples for e in out.entries)
            logits = self.runner.step(entries, commit=False, decode_graph=decode_only)
            t2 = time.perf_counter()
            if rows:
                sampled = self.sampler.sample(logits, [r.params for r in rows],
                                              [r.sampling_counter for r in rows],
                                              [r.tokens if r.params.repetition_penalty != 1.0 else ()
                                               for r in rows])
            else:
                torch.cuda.current_stream().synchronize()
        else:
            t2 = time.perf_counter()
        t3 = time.perf_counter()
        self.scheduler.process_outputs(out, sampled)
        t4 = time.perf_counter()
        p = self.profile
        p["schedule"] += t1 - t0
        p["forward"] += t2 - t1
        p["sample"] += t3 - t2
        p["process"] += t4 - t3
        p["steps"] += 1
        return self.scheduler.pop_finished()

    # ------------------------------------------------------------------ whole requests
    def generate(self, prompts: Sequence[Sequence[int]],
                 sampling_params: Union[SamplingParams, Sequence[SamplingParams], None] = None
                 ) -> List[GenerationResult]:
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params or SamplingParams()] * len(prompts)
        if len(sampling_params) != len(prompts):
            raise ValueError("one SamplingParams per prompt, or one for all")
        reqs = [self.add_request(p, sp) for p, sp in zip(prompts, sampling_params)]
        finished: Dict[int, Request] = {r.request_id: r for r in self.scheduler.pop_finished()}
        while self.scheduler.has_active_requests():
            for r in self.step():
                finished[r.request_id] = r
        for r in self.scheduler.pop_finished():
            finished[r.request_id] = r
        return [GenerationResult(r.request_id, list(r.prompt), list(r.outputs), r.finish_reason,
                                 r.preemptions) for r in reqs]


def generate(model, prompts, sampling_params=None, **engine_args) -> List[List[int]]:
    """One call: build an engine for ``model`` and return the generated token ids."""
    eng = Engine(model, **engine_args)
    return [r.output_tokens for r in eng.generate(prompts, sampling_params)]
