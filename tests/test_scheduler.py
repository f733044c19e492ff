"""The scheduler's decisions with scripted sampled tokens and no model (no GPU), in the
manner of the reference's scheduler test (test/test_scheduler_radix_cache.cpp:50-135):
token budget, portion caps, decode first, admission order, finishing, and what happens
when pages run out (preempt and recompute; fail what can never run)."""
import pytest

from paged_batch_engine_b200.cache import CacheManager, KVGroupSpec
from paged_batch_engine_b200.engine.scheduler import Scheduler, SchedulerConfig
from paged_batch_engine_b200.sampling.params import SamplingParams, request_sample_uniform


def make(pages=64, page=4, **cfg):
    m = CacheManager([KVGroupSpec((0, 1), 2, 16)], page, pages, max_requests=cfg.pop("slots", 16))
    defaults = dict(max_num_seqs=8, max_num_batched_tokens=16, prefill_chunk_cap=8)
    defaults.update(cfg)
    return m, Scheduler(SchedulerConfig(**defaults), m, eos_token_ids=[99])


def drive(s, token_fn=lambda req: 7, max_steps=500):
    """Runs steps with a scripted sampler; returns the list of per-step entry summaries."""
    log = []
    for _ in range(max_steps):
        if not s.has_active_requests():
            break
        out = s.schedule_step()
        log.append([(e.request.request_id, len(e.tokens), e.samples) for e in out.entries])
        s.process_outputs(out, [token_fn(e.request) for e in out.entries if e.samples])
        s.cache.check_invariants()
    assert not s.has_active_requests()
    return log


def test_prompt_is_cut_under_budget_and_cap_then_decoded():
    m, s = make()
    r = s.add_request(list(range(1, 21)), SamplingParams(max_new_tokens=3))
    log = drive(s)
    assert log[:3] == [[(0, 8, False)], [(0, 8, False)], [(0, 4, True)]]      # cap 8, last portion samples
    assert log[3:] == [[(0, 1, True)], [(0, 1, True)]]
    assert r.outputs == [7, 7, 7] and r.finish_reason == "length" and r.status == "finished"
    assert m.num_live_requests == 0 and m.num_free_pages() == 64


def test_decodes_first_then_running_prompts_then_new_requests():
    m, s = make(max_num_batched_tokens=10, prefill_chunk_cap=6)
    a = s.add_request([1] * 3, SamplingParams(max_new_tokens=50))
    drive_one = lambda: s.process_outputs(o, [7] * sum(e.samples for e in o.entries))
    o = s.schedule_step(); drive_one()                       # a's prompt; a now decodes
    b = s.add_request([2] * 14, SamplingParams(max_new_tokens=2))
    c = s.add_request([3] * 5, SamplingParams(max_new_tokens=2))
    o = s.schedule_step()
    assert [(e.request.request_id, len(e.tokens)) for e in o.entries] == [(0, 1), (1, 6), (2, 3)]
    assert o.num_decode == 1 and o.total_tokens == 10        # the budget is used up exactly
    drive_one()
    o = s.schedule_step()
    # decode row first, then the running prompts in order, each within cap and budget
    assert [(e.request.request_id, len(e.tokens), e.samples) for e in o.entries] == \
        [(0, 1, True), (1, 6, False), (2, 2, True)]
    drive_one()
    o = s.schedule_step()
    assert [(e.request.request_id, len(e.tokens), e.samples) for e in o.entries] == \
        [(0, 1, True), (2, 1, True), (1, 2, True)]


def test_max_num_seqs_and_fifo_admission():
    m, s = make(max_num_seqs=2)
    reqs = [s.add_request([5] * 4, SamplingParams(max_new_tokens=2)) for _ in range(4)]
    o = s.schedule_step()
    assert [e.request.request_id for e in o.entries] == [0, 1]
    s.process_outputs(o, [7, 7])
    log = drive(s)
    order = [r.request_id for r in s.pop_finished()]
    assert order == [0, 1, 2, 3]


def test_eos_min_new_tokens_and_ignore_eos():
    m, s = make()
    a = s.add_request([1, 2], SamplingParams(max_new_tokens=10))
    b = s.add_request([1, 2], SamplingParams(max_new_tokens=10, min_new_tokens=3))
    c = s.add_request([1, 2], SamplingParams(max_new_tokens=4, ignore_eos=True))
    drive(s, token_fn=lambda r: 99)
    assert a.outputs == [] and a.finish_reason == "stop" and a.generated == 1    # EOS is not part of the output
    assert b.finish_reason == "stop" and b.generated == 4 and b.outputs == [99, 99, 99]
    assert c.finish_reason == "length" and c.outputs == [99] * 4


def test_portion_is_cut_to_the_free_pages():
    m, s = make(pages=5, page=4, max_num_batched_tokens=64, prefill_chunk_cap=64)
    a = s.add_request([1] * 9, SamplingParams(max_new_tokens=2))      # 3 pages
    o = s.schedule_step(); s.process_outputs(o, [7])
    b = s.add_request([2] * 13, SamplingParams(max_new_tokens=1))     # needs 4 pages, 2 are free
    o = s.schedule_step()
    assert [(e.request.request_id, len(e.tokens)) for e in o.entries] == [(0, 1), (1, 8)]
    s.process_outputs(o, [7])                                         # a finishes, pages come back
    o = s.schedule_step()
    assert [(e.request.request_id, len(e.tokens), e.samples) for e in o.entries] == [(1, 5, True)]


def test_decode_without_a_page_is_preempted_and_recomputed():
    m, s = make(pages=4, page=4, max_num_batched_tokens=64, prefill_chunk_cap=64)
    a = s.add_request([1] * 7, SamplingParams(max_new_tokens=8))
    b = s.add_request([2] * 7, SamplingParams(max_new_tokens=3))
    seen = []
    for _ in range(200):
        if not s.has_active_requests():
            break
        o = s.schedule_step()
        seen.append(([(e.request.request_id, len(e.tokens), e.samples) for e in o.entries], list(o.preempted)))
        s.process_outputs(o, [40 + e.request.generated for e in o.entries if e.samples])
        m.check_invariants()
    assert not s.has_active_requests()
    assert s.metrics["preemptions"] >= 1 and any(p for _, p in seen)
    victim = a if a.preemptions else b
    # the preempted request came back with its prompt and outputs as one portion to recompute
    assert any(n > 7 for entries, _ in seen for rid, n, _ in entries if rid == victim.request_id)
    # every request still received exactly its tokens, in order, despite the recomputation
    assert a.outputs == [40 + i for i in range(8)] and b.outputs == [40 + i for i in range(3)]
    assert a.finish_reason == b.finish_reason == "length"
    assert m.num_free_pages() == 4 and m.num_live_requests == 0


def test_preempted_request_waits_until_its_whole_context_fits():
    m, s = make(pages=12, page=4, max_num_batched_tokens=64, prefill_chunk_cap=64)
    a = s.add_request([1] * 10, SamplingParams(max_new_tokens=30))
    b = s.add_request([2] * 10, SamplingParams(max_new_tokens=30))
    running_when_admitted = []
    for _ in range(400):
        if not s.has_active_requests():
            break
        o = s.schedule_step()
        for e in o.entries:
            if e.request.preemptions and len(e.tokens) > 1 and e.request.computed == 0:
                # admitted again: room for all its tokens plus the next one was free
                need = (e.request.target + 1 + 3) // 4
                running_when_admitted.append(need)
        s.process_outputs(o, [7] * sum(e.samples for e in o.entries))
    assert not s.has_active_requests()
    assert s.metrics["preemptions"] >= 1 and running_when_admitted
    assert len(a.outputs) == 30 and len(b.outputs) == 30
    assert a.status == b.status == "finished" and m.num_free_pages() == 12


def test_requests_that_can_never_run_fail_instead_of_waiting():
    m, s = make(pages=3, page=4)
    too_long = s.add_request([1] * 13)
    assert too_long.status == "failed" and too_long.finish_reason == "prompt_exceeds_kv_capacity"
    empty = s.add_request([])
    assert empty.status == "failed"
    # fits alone but grows beyond the pool while decoding: preempted, then can never come back
    r = s.add_request([1] * 10, SamplingParams(max_new_tokens=20))
    drive(s)
    assert r.status == "failed" and r.finish_reason == "preempted_recompute_exceeds_kv_capacity"
    assert r.outputs == [7] * 3                     # 10 + 2 fed tokens filled the 12 slots
    assert m.num_free_pages() == 3 and m.num_live_requests == 0
    assert [x.request_id for x in s.pop_finished()] == [0, 1, 2]


def test_stalled_prompts_do_not_deadlock():
    m, s = make(pages=4, page=4, max_num_seqs=2, max_num_batched_tokens=12, prefill_chunk_cap=6)
    a = s.add_request([1] * 12, SamplingParams(max_new_tokens=1))
    b = s.add_request([2] * 12, SamplingParams(max_new_tokens=1))
    drive(s)
    assert sorted([a.status, b.status]) == ["failed", "finished"]
    assert "prefill_stalled_kv_exhausted" in (a.finish_reason, b.finish_reason)
    assert m.num_free_pages() == 4


def test_no_request_slot_left_waits():
    m, s = make(slots=1)
    a = s.add_request([1] * 3, SamplingParams(max_new_tokens=2))
    b = s.add_request([1] * 3, SamplingParams(max_new_tokens=2))
    log = drive(s)
    assert all(len(step) == 1 for step in log) and a.outputs == b.outputs == [7, 7]


def test_long_prompt_threshold_and_cancel():
    m, s = make(long_prefill_token_threshold=3, prefill_chunk_cap=8)
    a = s.add_request([1] * 10, SamplingParams(max_new_tokens=1))
    o = s.schedule_step()
    assert len(o.entries[0].tokens) == 3
    s.process_outputs(o, [])
    s.cancel(a)
    assert a.finish_reason == "cancelled" and m.num_free_pages() == 64 and not s.has_active_requests()


def test_uniform_draws_depend_on_seed_and_counter_only():
    """test/test_request_progress.cpp:7-52: reorder and retry do not consume random state."""
    a = [request_sample_uniform(11, c) for c in range(5)]
    assert a == [request_sample_uniform(11, c) for c in range(5)]
    assert a != [request_sample_uniform(12, c) for c in range(5)]
    assert all(0.0 <= u < 1.0 for u in a) and len(set(a)) == 5
    p = SamplingParams(temperature=-1, top_p=7, top_k=-3, max_new_tokens=0, min_new_tokens=9).normalized()
    assert (p.temperature, p.top_p, p.top_k, p.max_new_tokens, p.min_new_tokens) == (0.0, 1.0, 0, 1, 1)
    assert p.is_greedy and not SamplingParams(top_k=5).is_greedy


def drive_ahead(s, token_fn, max_steps=500):
    """As the engine pipelines decode steps: the step after a running one is scheduled before
    the running one's tokens are processed, whenever the scheduler allows it."""
    log, pending = [], None
    for _ in range(max_steps):
        if pending is None and not s.has_active_requests():
            break
        if pending is not None:
            ahead = s.schedule_ahead(pending)
            s.process_outputs(pending, [token_fn(e.request) for e in pending.entries if e.samples])
            s.cache.check_invariants()
            pending = ahead
            if ahead is not None:
                log.append(("ahead", [e.request.request_id for e in ahead.entries]))
                continue
        out = s.schedule_step()
        log.append(("step", [(e.request.request_id, len(e.tokens)) for e in out.entries]))
        pending = out if out.entries else None
    assert not s.has_active_requests()
    return log


def test_decode_steps_scheduled_one_ahead_give_the_same_tokens():
    """Two requests decode together; steps are scheduled ahead until a length limit is one
    token away, an end-of-sequence token drops the token computed in vain, and counters,
    outputs and pages end as without the pipeline."""
    outs = []
    for ahead in (False, True):
        m, s = make()
        script = {0: iter([5, 6, 99, 1, 1, 1]), 1: iter(range(10, 40))}
        a = s.add_request([1, 2, 3], SamplingParams(max_new_tokens=6))              # stops on 99 (EOS) as 3rd token
        b = s.add_request([4, 5], SamplingParams(max_new_tokens=7, ignore_eos=True))
        fn = lambda req: next(script[req.request_id])
        log = drive_ahead(s, fn) if ahead else drive(s, fn)
        outs.append((a.outputs, a.finish_reason, a.sampling_counter, b.outputs, b.finish_reason, b.sampling_counter))
        assert m.num_live_requests == 0 and m.num_free_pages() == 64
        if ahead:
            assert s.metrics["ahead_steps"] >= 3
            assert s.metrics["dropped_tokens"] == 1            # a's token after its end-of-sequence
            assert any(kind == "ahead" for kind, _ in log)
    # the scripted sampler hands a one more token in the pipelined run (the dropped one), so b's
    # tokens are the same and a's are cut at the same place
    assert outs[0][:3] == outs[1][:3] == ([5, 6], "stop", 3)
    assert outs[0][3:] == outs[1][3:] and len(outs[0][3]) == 7


def test_nothing_is_scheduled_ahead_when_it_could_be_wrong():
    m, s = make(pages=3, page=4)
    r = s.add_request([1, 2, 3], SamplingParams(max_new_tokens=50, ignore_eos=True))
    o = s.schedule_step()
    assert s.schedule_ahead(o) is None                         # a prompt portion: not a decode step
    s.process_outputs(o, [7])
    o = s.schedule_step()                                      # first decode step (position 3)
    assert [len(e.tokens) for e in o.entries] == [1]
    w = s.add_request([9], SamplingParams(max_new_tokens=2))
    assert s.schedule_ahead(o) is None                         # a request waits to be admitted
    s.cancel(w)
    s.pop_finished()
    nxt = s.schedule_ahead(o)
    assert nxt is not None and nxt.entries[0].counter == r.sampling_counter + 1
    assert m.reserved_len(r.handle) == m.context_len(r.handle) + 2
    s.process_outputs(o, [7])
    s.process_outputs(nxt, [7])
    assert r.outputs == [7, 7, 7] and r.sampling_counter == 3 and m.context_len(r.handle) == 5
    # pages: 3 x 4 tokens; at 11 tokens reserved the next step ahead finds no page and gives back
    # what it took, the usual step then preempts or fails as it decides
    while True:
        o = s.schedule_step()
        if not o.entries:
            break
        before = m.reserved_len(r.handle)
        nxt = s.schedule_ahead(o)
        if nxt is None:
            assert m.reserved_len(r.handle) == before
            s.process_outputs(o, [7])
            if r.done:
                break
            continue
        s.process_outputs(o, [7])
        s.process_outputs(nxt, [7])
    m.check_invariants()
    p = SamplingParams(max_new_tokens=4, repetition_penalty=1.3)
    m2, s2 = make()
    q = s2.add_request([1, 2], p)
    o = s2.schedule_step(); s2.process_outputs(o, [7])
    o = s2.schedule_step()
    # a repetition penalty does not keep a step from being scheduled ahead: the sampler keeps the
    # request's seen tokens on the device
    assert s2.schedule_ahead(o) is not None


def test_sizes_of_captured_decode_steps_and_key_splits():
    """Captured decode steps come in powers of two and, from 24 rows on, the sizes half-way; the
    padding never exceeds a third of the rows from 16 requests on.  Key splits are 512 keys for
    at most four requests (the first bucket edge) and 256 beyond, by the bucket as by the count."""
    from paged_batch_engine_b200.engine.batch import choose_split_keys
    from paged_batch_engine_b200.engine.graphs import _batch_bucket
    assert [_batch_bucket(n) for n in (1, 2, 3, 5, 8, 9, 16, 17, 24, 25, 32, 33, 48, 49, 64, 65, 96, 97, 128, 200)] == \
        [1, 2, 4, 8, 8, 16, 16, 24, 24, 32, 32, 48, 48, 64, 64, 96, 96, 128, 128, 256]
    for n in range(1, 600):
        b = _batch_bucket(n)
        assert b >= n and (n < 16 or (b - n) * 3 <= b)
        assert choose_split_keys(n) == choose_split_keys(b)
    assert choose_split_keys(4) == 512 and choose_split_keys(5) == 256


def test_request_metric_and_final_summary_records():
    """Time to first token, the mean token gap and the latency as the reference defines them
    (sequence_state.h:140-165), and the run's summary from the scheduler's counters."""
    import time
    from paged_batch_engine_b200.engine import metrics
    m, s = make()
    a = s.add_request(list(range(1, 12)), SamplingParams(max_new_tokens=4))
    b = s.add_request([5, 6], SamplingParams(max_new_tokens=1))
    c = s.add_request([], SamplingParams(max_new_tokens=1))              # fails at once: empty prompt
    t0 = time.perf_counter()
    drive(s, token_fn=lambda req: (time.sleep(0.002), 7)[1])
    wall = time.perf_counter() - t0
    assert a.arrival_time <= a.first_token_time <= a.last_token_time == a.finished_time
    assert len(a.token_times) == a.generated == 4 and len(b.token_times) == 1
    assert metrics.ttft_ms(a) > 0 and metrics.latency_ms(a) >= metrics.ttft_ms(a)
    gap = (a.last_token_time - a.first_token_time) * 1e3 / 3
    assert abs(metrics.itl_ms(a) - gap) < 1e-9 and metrics.itl_ms(b) == 0.0
    line = metrics.request_metric_line(a)
    assert line.startswith("REQUEST_METRIC client_request_id=0 status=ok prompt_tokens=11 generated_tokens=4 "
                           "output_tokens=4 ttft_ms=") and " finish_reason=length" in line
    assert "status=failed" in metrics.request_metric_line(c) and "finish_reason=empty_prompt" in metrics.request_metric_line(c)
    summ = metrics.final_summary([a, b, c], s.metrics, dict(steps=s.metrics["steps"], schedule=0.01), wall)
    assert summ["completed_requests"] == 2 and summ["failed_requests"] == 1
    assert summ["total_prefill_tokens"] == 13 and summ["total_decode_tokens"] == 3
    assert summ["total_steps"] == s.metrics["steps"] and summ["decode_only_steps"] == 3
    assert summ["token_gap_count"] == 3 and summ["token_gap_p50_ms"] > 0
    assert summ["ttft_p50_ms"] <= summ["ttft_p99_ms"] and summ["throughput_tps"] == pytest.approx(5 / wall)
    text = metrics.final_summary_line(summ)
    assert text.startswith("FINAL_SUMMARY total_steps=") and " itl_ms=" in text and " latency_p95_ms=" in text
    assert metrics.percentile([1.0, 2.0, 3.0, 4.0], 0.5) == 2.5 and metrics.percentile([], 0.9) == 0.0
