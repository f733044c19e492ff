"""Continuous batching under a token budget: admits requests, cuts prompts into portions,
decodes, finishes and frees; preempts by recomputation when pages run out.

It follows the reference's ``serving::Scheduler`` (infMain/source/serving/scheduler.cpp):
one step = (1) every running request that is decoding gets one row, in order, while the
budget lasts; one that cannot get a page is preempted: everything it holds is freed and it
goes back to the waiting queue to be recomputed (:783-804, :926-976); (2) running requests
still in their prompt get a portion min(remaining, budget, cap), further cut to what the
free pages can hold (:806-831, :586-609, :23-34); (3) the head of the waiting queue is
admitted while there is budget and room for another request, stopping at the first that
cannot start (:833-873); a request that was preempted is admitted only when its whole
context plus one token fits (:1043-1073); (4) if nothing could be scheduled, a request
that can never run is failed instead of waiting for ever (:1075-1186).

It decides with the cache manager only and never touches the device, so its decisions are
tested without a GPU by scripting the sampled tokens.
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, List, Optional, Sequence, Tuple

from ..cache.manager import CacheManager
from ..sampling.params import SamplingParams


@dataclass
class SchedulerConfig:
    max_num_seqs: int = 256              # requests running at a time
    max_num_batched_tokens: int = 2048   # rows per step
    prefill_chunk_cap: int = 512         # longest prompt portion per request and step
    long_prefill_token_threshold: int = 0  # >0: prompts with more remaining tokens get portions of at most this
    max_model_len: int = 0               # >0: a request stops when its context reaches this


@dataclass
class Request:
    request_id: int
    prompt: List[int]
    params: SamplingParams
    outputs: List[int] = field(default_factory=list)
    handle: Optional[int] = None
    computed: int = 0                 # tokens whose keys and values are in the cache
    scheduled: int = 0                # tokens in flight this step
    generated: int = 0                # sampled tokens, EOS included
    sampling_counter: int = 0
    status: str = "waiting"           # waiting, running, preempted, finished, failed
    recompute: bool = False
    ready_step: int = 0
    finish_reason: str = ""
    preemptions: int = 0
    # host clock (time.perf_counter) of arrival, of every token as the host learned of it, and
    # of the end: what time to first token, token gaps and latency are made from
    arrival_time: Optional[float] = None
    token_times: List[float] = field(default_factory=list)
    finished_time: Optional[float] = None

    @property
    def first_token_time(self) -> Optional[float]:
        return self.token_times[0] if self.token_times else None

    @property
    def last_token_time(self) -> Optional[float]:
        return self.token_times[-1] if self.token_times else None

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.outputs

    def token_slice(self, lo: int, hi: int) -> List[int]:
        """tokens[lo:hi] without building the whole list (called for every row of every step)."""
        n = len(self.prompt)
        if hi <= n:
            return self.prompt[lo:hi]
        if lo >= n:
            return self.outputs[lo - n:hi - n]
        return self.prompt[lo:] + self.outputs[:hi - n]

    @property
    def target(self) -> int:
        """Tokens that must be in the cache before the next token can be sampled."""
        return len(self.prompt) + len(self.outputs)

    @property
    def remaining(self) -> int:
        return self.target - self.computed

    @property
    def is_decode(self) -> bool:
        return self.generated > 0 and not self.recompute and self.remaining == 1

    @property
    def done(self) -> bool:
        return self.status in ("finished", "failed")


@dataclass
class ScheduledEntry:
    request: Request
    tokens: List[int]
    samples: bool                      # the portion ends the known tokens: its last row is sampled
    counter: Optional[int] = None      # the request's sampling counter for this row, when it is not
    #                                    the request's current one (a step scheduled ahead)


@dataclass
class SchedulerOutput:
    entries: List[ScheduledEntry] = field(default_factory=list)
    num_decode: int = 0
    preempted: List[int] = field(default_factory=list)

    @property
    def total_tokens(self) -> int:
        return sum(len(e.tokens) for e in self.entries)


class Scheduler:
    def __init__(self, config: SchedulerConfig, cache: CacheManager, eos_token_ids: Sequence[int] = ()):
        if config.max_num_seqs <= 0 or config.max_num_batched_tokens <= 0 or config.prefill_chunk_cap <= 0:
            raise ValueError("scheduler limits must be positive")
        self.config, self.cache = config, cache
        self.eos = set(int(t) for t in eos_token_ids)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.finished: List[Request] = []
        self.step_index = 0
        self._next_id = 0
        self.metrics = dict(steps=0, preemptions=0, decode_tokens=0, prefill_tokens=0, no_progress_steps=0,
                            failed=0, ahead_steps=0, dropped_tokens=0, decode_only_steps=0,
                            max_waiting_queue=0, max_running_queue=0)

    # ------------------------------------------------------------------ requests in and out
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None) -> Request:
        req = Request(self._next_id, [int(t) for t in prompt], (params or SamplingParams()).normalized())
        req.arrival_time = time.perf_counter()
        self._next_id += 1
        if not req.prompt:
            self._fail(req, "empty_prompt")
            return req
        if len(req.prompt) > self.cache.capacity_tokens():
            self._fail(req, "prompt_exceeds_kv_capacity")          # scheduler.cpp:161-171
            return req
        self.waiting.append(req)
        return req

    def has_active_requests(self) -> bool:
        return bool(self.waiting or self.running)

    def pop_finished(self) -> List[Request]:
        out, self.finished = self.finished, []
        return out

    def cancel(self, req: Request) -> None:
        if req.done:
            return
        self._release(req)
        if req in self.running:
            self.running.remove(req)
        if req in self.waiting:
            self.waiting.remove(req)
        req.status, req.finish_reason = "finished", "cancelled"
        req.finished_time = time.perf_counter()
        self.finished.append(req)

    # ------------------------------------------------------------------ one step
    def schedule_step(self) -> SchedulerOutput:
        self.step_index += 1
        self.metrics["steps"] += 1
        out = SchedulerOutput()
        budget = self.config.max_num_batched_tokens
        budget = self._schedule_decodes(out, budget)
        budget = self._schedule_running_prefills(out, budget)
        self._requeue_preempted()
        budget = self._admit_waiting(out, budget)
        if not out.entries:
            self.metrics["no_progress_steps"] += 1
            self._handle_no_progress()
        self.metrics["decode_tokens"] += out.num_decode
        self.metrics["prefill_tokens"] += out.total_tokens - out.num_decode
        if out.entries and out.num_decode == len(out.entries):
            self.metrics["decode_only_steps"] += 1
        self.metrics["max_waiting_queue"] = max(self.metrics["max_waiting_queue"], len(self.waiting))
        self.metrics["max_running_queue"] = max(self.metrics["max_running_queue"], len(self.running))
        return out

    def _schedule_decodes(self, out: SchedulerOutput, budget: int) -> int:
        limit = min(budget, self.config.max_num_seqs - out.num_decode)
        decoding = [r for r in self.running if r.is_decode][:max(limit, 0)]
        if not decoding:
            return budget
        # one call reserves a slot for every decoding request; from the first that finds no
        # page on, go one by one, because a preemption gives pages back to those after it
        ok = self.cache.reserve_many([r.handle for r in decoding], 1)
        first_bad = ok.index(False) if False in ok else len(ok)
        for i, req in enumerate(decoding):
            if i < first_bad:
                got = True
            elif i == first_bad:
                got = False
            else:
                got = ok[i] or self.cache.reserve(req.handle, 1)
            if not got:
                self._preempt(req, out)
                continue
            req.scheduled = 1
            out.entries.append(ScheduledEntry(req, req.token_slice(req.computed, req.computed + 1), True))
            out.num_decode += 1
            budget -= 1
        return budget

    def _chunk_for(self, req: Request, budget: int) -> int:
        cap = self.config.prefill_chunk_cap
        thr = self.config.long_prefill_token_threshold
        if thr > 0 and req.remaining > thr:
            cap = min(cap, thr)
        return min(req.remaining, budget, cap)

    def _schedule_running_prefills(self, out: SchedulerOutput, budget: int) -> int:
        for req in self.running:
            if budget <= 0:
                break
            if req.status != "running" or req.is_decode or req.scheduled:
                continue
            chunk = min(self._chunk_for(req, budget), self.cache.max_appendable_tokens(req.handle))
            if chunk <= 0:
                continue
            if not self.cache.reserve(req.handle, chunk):
                continue
            self._append_prefill(req, chunk, out)
            budget -= chunk
        return budget

    def _admit_waiting(self, out: SchedulerOutput, budget: int) -> int:
        while self.waiting and budget > 0 and len(self.running) < self.config.max_num_seqs:
            req = self.waiting[0]
            if req.ready_step > self.step_index:
                break
            handle = self.cache.add_request(req.request_id)
            if handle is None:
                break
            desired = self._chunk_for(req, budget)
            ok = desired > 0
            if ok and req.recompute and not self.cache.can_reserve(handle, req.target + 1):
                ok = False              # would be preempted again at once (scheduler.cpp:1043-1073)
            chunk = min(desired, self.cache.max_appendable_tokens(handle)) if ok else 0
            if chunk <= 0 or not self.cache.reserve(handle, chunk):
                self.cache.free(handle)
                break
            self.waiting.popleft()
            req.handle, req.status, req.computed = handle, "running", 0
            self.running.append(req)
            self._append_prefill(req, chunk, out)
            budget -= chunk
        return budget

    def _append_prefill(self, req: Request, chunk: int, out: SchedulerOutput) -> None:
        toks = req.token_slice(req.computed, req.computed + chunk)
        req.scheduled = chunk
        out.entries.append(ScheduledEntry(req, toks, req.computed + chunk == req.target))

    # ------------------------------------------------------------------ running out of pages
    def _preempt(self, req: Request, out: SchedulerOutput) -> None:
        """Recompute later: give back everything now (scheduler.cpp:926-976)."""
        self._release(req)
        req.computed, req.scheduled = 0, 0
        req.recompute = True
        req.status = "preempted"
        req.preemptions += 1
        req.ready_step = self.step_index + 1
        self.metrics["preemptions"] += 1
        out.preempted.append(req.request_id)

    def _requeue_preempted(self) -> None:
        moved = [r for r in self.running if r.status == "preempted"]
        if moved:
            self.running = [r for r in self.running if r.status != "preempted"]
            for r in moved:
                r.status = "waiting"
                self.waiting.append(r)

    def _release(self, req: Request) -> None:
        if req.handle is not None and self.cache.is_live(req.handle):
            self.cache.free(req.handle)
        req.handle = None

    def _fail(self, req: Request, reason: str) -> None:
        self._release(req)
        req.status, req.finish_reason = "failed", reason
        req.finished_time = time.perf_counter()
        self.metrics["failed"] += 1
        self.finished.append(req)

    def _handle_no_progress(self) -> None:
        """Nothing could run.  If nothing is running either, the head of the waiting queue
        will never fit: fail it.  If only stalled prompt portions are running, fail the
        first of them (scheduler.cpp:1075-1186)."""
        if self.waiting and not self.running:
            req = self.waiting[0]
            if req.ready_step > self.step_index:
                return
            self.waiting.popleft()
            self._fail(req, "preempted_recompute_exceeds_kv_capacity" if req.recompute
                       else "prefill_cannot_start")
            return
        stalled = [r for r in self.running if not r.is_decode]
        if stalled and not any(r.is_decode for r in self.running):
            req = stalled[0]
            self.running.remove(req)
            self._fail(req, "prefill_stalled_kv_exhausted")

    # ------------------------------------------------------------------ one step ahead
    def schedule_ahead(self, prev: SchedulerOutput) -> Optional[SchedulerOutput]:
        """The step after ``prev`` while ``prev`` still runs on the device and its tokens are
        not known: possible when ``prev`` is decoded tokens only, nothing waits to be admitted,
        and every request of ``prev`` goes on whatever it samples now (its length limits are
        not reached by that token, and sampling needs none of its tokens on the host).  Only an
        end-of-sequence token cannot be foreseen: a request that stops on ``prev``'s token has
        one token computed in vain, which ``process_outputs`` drops.  The entries carry
        placeholder token ids (the step takes them from the device) and keep ``prev``'s order.
        Returns None when the step cannot be scheduled ahead; nothing is changed then."""
        if not prev.entries or prev.preempted or self.waiting or len(prev.entries) != len(self.running):
            return None
        limit = self.config.max_model_len
        for e in prev.entries:
            req, p = e.request, e.request.params
            if (len(e.tokens) != 1 or not e.samples or req.done or req.status != "running" or req.recompute
                    or req.generated + 1 >= p.max_new_tokens
                    or (limit > 0 and req.target + 1 >= limit)):
                return None
        handles = [e.request.handle for e in prev.entries]
        ok = self.cache.reserve_many(handles, 1)
        if not all(ok):
            for h, got in zip(handles, ok):                 # give back what was taken: the usual step decides
                if got:
                    self.cache.truncate(h, self.cache.reserved_len(h) - 1)
            return None
        self.step_index += 1
        self.metrics["steps"] += 1
        self.metrics["ahead_steps"] += 1
        self.metrics["decode_only_steps"] += 1
        out = SchedulerOutput()
        for e in prev.entries:
            out.entries.append(ScheduledEntry(e.request, [0], True, counter=e.request.sampling_counter + 1))
        out.num_decode = len(out.entries)
        self.metrics["decode_tokens"] += out.num_decode
        return out

    # ------------------------------------------------------------------ after the step
    def process_outputs(self, out: SchedulerOutput, sampled: Sequence[int]) -> None:
        """``sampled``: one token for each entry with ``samples``, in entry order.  Entries of
        requests that ended meanwhile (a step scheduled ahead of the token that stopped them, a
        cancellation) are dropped with their tokens."""
        it = iter(sampled)
        live = [e for e in out.entries if not e.request.done and e.request.handle is not None]
        if live:
            self.cache.commit_many([e.request.handle for e in live], [len(e.tokens) for e in live])
        for e in out.entries:
            req = e.request
            if req.done or req.handle is None:
                if e.samples:
                    next(it, None)
                    self.metrics["dropped_tokens"] += 1
                continue
            req.computed += len(e.tokens)
            req.scheduled = 0
            if e.samples:
                if req.recompute:
                    req.recompute = False
                self._record_token(req, int(next(it)))
        leftover = list(it)
        if leftover:
            raise ValueError(f"{len(leftover)} sampled tokens belong to no entry")
        done = [r for r in self.running if r.done]
        if done:
            self.running = [r for r in self.running if not r.done]
            for r in done:
                self._release(r)
                self.finished.append(r)

    def _record_token(self, req: Request, token: int) -> None:
        """scheduler.cpp:84-107: EOS stops the request unless ignored or too early and is
        not part of the output; the token budget stops it after max_new_tokens."""
        req.generated += 1
        req.sampling_counter += 1
        now = time.perf_counter()
        req.token_times.append(now)
        is_eos = token in self.eos
        p = req.params
        if is_eos and not p.ignore_eos and req.generated > p.min_new_tokens:
            req.status, req.finish_reason, req.finished_time = "finished", "stop", now
            return
        req.outputs.append(token)
        if req.generated >= p.max_new_tokens:
            req.status, req.finish_reason, req.finished_time = "finished", "length", now
        elif self.config.max_model_len > 0 and req.target >= self.config.max_model_len:
            req.status, req.finish_reason, req.finished_time = "finished", "length", now
