"""Generation through the Python entry point and the command line: greedy tokens equal
the plain implementation's; sampled tokens equal the reference's sampling algorithm on
plain logits; captured decode graphs, few pages (preemption and recomputation) and
batching do not change the tokens."""
import json
import os
import subprocess

import pytest
import torch

from tests.helpers import TINY, load_plain
from tests.plain import plain_qwen2 as plain

pytestmark = pytest.mark.gpu
ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))


def prompts_for(vocab, lens, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab - 8, (n,), generator=g).tolist() for n in lens]


def engine(folder, dtype, page, **kw):
    from paged_batch_engine_b200 import Engine
    kw.setdefault("num_pages", 64)
    kw.setdefault("max_num_batched_tokens", 32)
    kw.setdefault("prefill_chunk_cap", 16)
    return Engine(folder, dtype=dtype, page_size=page, **kw)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_generation_equals_plain(tiny_folders, name):
    from paged_batch_engine_b200 import SamplingParams
    cfg, _, page, _ = TINY[name]
    folder = tiny_folders[name]
    pcfg, w = load_plain(folder)
    prompts = prompts_for(cfg["vocab_size"], [5, 17, 33] if name == "A" else [1, 9, 40, 71])
    eng = engine(folder, "float32", page)
    res = eng.generate(prompts, SamplingParams(max_new_tokens=8, ignore_eos=True))
    for p, r in zip(prompts, res):
        assert r.output_tokens == plain.greedy_generate(pcfg, w, p, 8), (name, len(p))
        assert r.finish_reason == "length" and r.prompt_tokens == p
    assert eng.runner.graphs.replays > 0                  # decode steps went through captured graphs
    assert eng.runner.cache.num_live_requests == 0
    # the same without graphs, and one prompt at a time
    eng2 = engine(folder, "float32", page, use_cuda_graphs=False)
    for p, r in zip(prompts, res):
        assert eng2.generate([p], SamplingParams(max_new_tokens=8, ignore_eos=True))[0].output_tokens == r.output_tokens


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_steps_one_ahead_change_no_token(tiny_folders, dtype):
    """Decode steps pipelined one deep (the next step launched before this step's tokens are
    read, its ids fed on the device) against the same engine without the pipeline: greedy and
    seeded temperature sampling, requests of different lengths, and a request that stops on an
    end-of-sequence token in the middle (one token is computed in vain and dropped)."""
    from paged_batch_engine_b200 import SamplingParams
    cfg, _, page, _ = TINY["B"]
    folder = tiny_folders["B"]
    prompts = prompts_for(cfg["vocab_size"], [3, 11, 26, 7], seed=21)
    params = [SamplingParams(max_new_tokens=14), SamplingParams(max_new_tokens=9, temperature=0.8, seed=5),
              SamplingParams(max_new_tokens=20, temperature=1.1, top_k=12, seed=9), SamplingParams(max_new_tokens=17)]
    plain_run = engine(folder, dtype, page, decode_ahead=False).generate(prompts, params)
    stop = plain_run[0].output_tokens[5]                  # make request 0 stop there
    results = []
    for ahead in (False, True):
        eng = engine(folder, dtype, page, decode_ahead=ahead)
        eng.scheduler.eos = {stop}
        res = eng.generate(prompts, params)
        results.append([(r.output_tokens, r.finish_reason) for r in res])
        assert eng.runner.cache.num_live_requests == 0
        eng.runner.cache.check_invariants()
        if ahead:
            assert eng.scheduler.metrics["ahead_steps"] >= 5
            assert eng.scheduler.metrics["dropped_tokens"] >= 1
        else:
            assert eng.scheduler.metrics["ahead_steps"] == 0
    assert results[0] == results[1]
    assert results[0][0][1] == "stop" and len(results[0][0][0]) <= 5


def test_cancelling_a_request_while_its_step_runs(tiny_folders):
    """A request is cancelled while a decode step that holds it is still running (pipelined
    steps): its token is dropped, its pages go back, the others go on unchanged."""
    from paged_batch_engine_b200 import SamplingParams
    cfg, _, page, _ = TINY["A"]
    folder = tiny_folders["A"]
    prompts = prompts_for(cfg["vocab_size"], [6, 13, 4], seed=4)
    sp = SamplingParams(max_new_tokens=12, ignore_eos=True)
    want = engine(folder, "float32", page).generate(prompts, sp)
    eng = engine(folder, "float32", page)
    reqs = [eng.add_request(p, sp) for p in prompts]
    while len(reqs[1].outputs) < 4:
        eng.step()
    assert eng._pending is not None                        # a decode step is in flight
    eng.scheduler.cancel(reqs[1])
    while eng.has_unfinished_requests():
        eng.step()
    eng.drain()
    assert reqs[1].finish_reason == "cancelled" and reqs[1].outputs == want[1].output_tokens[:len(reqs[1].outputs)]
    assert reqs[0].outputs == want[0].output_tokens and reqs[2].outputs == want[2].output_tokens
    assert eng.runner.cache.num_live_requests == 0
    eng.runner.cache.check_invariants()


@pytest.mark.parametrize("name", ["A", "B"])
def test_bfloat16_greedy_tokens_are_plain_argmax_up_to_rounding(tiny_folders, name):
    from paged_batch_engine_b200 import SamplingParams
    cfg, _, page, _ = TINY[name]
    folder = tiny_folders[name]
    pcfg, w = load_plain(folder)
    prompts = prompts_for(cfg["vocab_size"], [9, 40], seed=3)
    res = engine(folder, "bfloat16", page).generate(prompts, SamplingParams(max_new_tokens=12, ignore_eos=True))
    for p, r in zip(prompts, res):
        seq = p + r.output_tokens
        logits = plain.forward_logits(pcfg, w, seq[:-1])
        for i, tok in enumerate(r.output_tokens):
            row = logits[len(p) - 1 + i]
            assert row.max() - row[tok] <= 0.02 * logits.abs().max(), (name, i)


@pytest.mark.parametrize("persistent", [False, True])
def test_many_requests_at_once(tiny_folders, monkeypatch, persistent):
    """Twenty requests decode together (captured steps of 32 rows), through either instance of
    the decode attention kernel (the persistent one is what a step of many work items takes: its
    threshold is set to zero here); every request must produce what it produces alone."""
    from paged_batch_engine_b200 import SamplingParams
    from paged_batch_engine_b200.csrc import ops as pbe_ops
    if persistent:
        monkeypatch.setattr(pbe_ops, "DECODE_BLOCK_ITEMS_PER_SM", 0)
    cfg, _, page, _ = TINY["C"]
    folder = tiny_folders["C"]
    prompts = prompts_for(cfg["vocab_size"], [3 + 5 * i for i in range(20)], seed=9)
    sp = SamplingParams(max_new_tokens=10, ignore_eos=True)
    for dtype in ("float32", "bfloat16"):
        eng = engine(folder, dtype, page, num_pages=256, max_num_seqs=32, max_num_batched_tokens=64)
        together = eng.generate(prompts, sp)
        assert eng.runner.graphs.replays > 0
        alone = engine(folder, dtype, page, num_pages=256)
        pcfg, w = load_plain(folder)
        for p, r in zip(prompts, together):
            if dtype == "float32":
                assert r.output_tokens == alone.generate([p], sp)[0].output_tokens
            else:
                seq = p + r.output_tokens
                logits = plain.forward_logits(pcfg, w, seq[:-1])
                for i, tok in enumerate(r.output_tokens):
                    row = logits[len(p) - 1 + i]
                    assert row.max() - row[tok] <= 0.02 * logits.abs().max()


def test_temperature_sampling_follows_the_reference_algorithm(tiny_folders):
    from paged_batch_engine_b200 import SamplingParams
    cfg, _, page, _ = TINY["B"]
    folder = tiny_folders["B"]
    pcfg, w = load_plain(folder)
    prompts = prompts_for(cfg["vocab_size"], [1, 9, 40, 71], seed=1)
    params = [SamplingParams(max_new_tokens=12, temperature=0.8, seed=100 + i, ignore_eos=True)
              for i in range(len(prompts))]
    params[2] = SamplingParams(max_new_tokens=12, temperature=1.1, top_k=20, top_p=0.9, seed=5,
                               repetition_penalty=1.3, ignore_eos=True)
    eng = engine(folder, "float32", page)
    res = eng.generate(prompts, params)
    again = engine(folder, "float32", page, max_num_batched_tokens=7, prefill_chunk_cap=5,
                   use_cuda_graphs=False).generate(prompts[::-1], params[::-1])[::-1]
    for p, sp, r, r2 in zip(prompts, params, res, again):
        assert r.output_tokens == r2.output_tokens          # batch order and portions do not matter
        seq = p + r.output_tokens
        logits = plain.forward_logits(pcfg, w, seq[:-1])
        for i, tok in enumerate(r.output_tokens):
            row = logits[len(p) - 1 + i].tolist()
            u = plain.request_sample_uniform(sp.seed, i)
            want = plain.sample_row(row, sp.temperature, sp.top_k, sp.top_p, sp.repetition_penalty,
                                    seen_tokens=seq[:len(p) + i], uniform=u)
            if tok != want:     # only when the draw sits on a boundary of the CDF
                pen = list(row)
                if sp.repetition_penalty != 1.0:
                    for t in set(seq[:len(p) + i]):
                        pen[t] = pen[t] / sp.repetition_penalty if pen[t] > 0 else pen[t] * sp.repetition_penalty
                iv = plain.sample_cdf_interval(pen, tok, sp.temperature, sp.top_k, sp.top_p)
                assert iv is not None and iv[0] - 1e-4 <= u <= iv[1] + 1e-4, (i, tok, want)
    assert any(len(set(r.output_tokens)) > 3 for r in res)     # it really sampled


def test_repetition_penalty_with_steps_in_flight_and_after_preemption(tiny_folders):
    """Requests with a repetition penalty decode through captured steps launched one ahead (their
    seen tokens live on the device) and give the tokens of an engine that reads every step before
    the next, also when pages run out and requests are recomputed."""
    from paged_batch_engine_b200 import SamplingParams
    cfg, _, page, _ = TINY["A"]
    folder = tiny_folders["A"]
    prompts = prompts_for(cfg["vocab_size"], [20, 25, 30, 18], seed=11)
    params = [SamplingParams(max_new_tokens=30, temperature=t, top_k=k, repetition_penalty=pen, seed=3 + i, ignore_eos=True)
              for i, (t, k, pen) in enumerate([(0.0, 0, 50.0), (0.9, 30, 1.2), (0.7, 0, 1.0), (1.2, 0, 0.8)])]
    plainly = engine(folder, "float32", page, num_pages=64, use_cuda_graphs=False).generate(prompts, params)
    ahead_engine = engine(folder, "float32", page, num_pages=64)
    ahead = ahead_engine.generate(prompts, params)
    assert ahead_engine.scheduler.metrics["ahead_steps"] > 0
    tight_engine = engine(folder, "float32", page, num_pages=9)
    tight = tight_engine.generate(prompts, params)
    assert tight_engine.scheduler.metrics["preemptions"] > 0
    for a, b, c in zip(plainly, ahead, tight):
        assert a.output_tokens == b.output_tokens == c.output_tokens
    assert not ahead_engine.sampler._slot_of and not tight_engine.sampler._slot_of      # rows given back
    # the greedy request with a penalty of 50 hardly ever repeats a token, the plain greedy one does
    free = engine(folder, "float32", page, num_pages=64).generate(prompts[:1], SamplingParams(max_new_tokens=30, ignore_eos=True))
    assert len(set(ahead[0].output_tokens)) >= 25 > len(set(free[0].output_tokens))


def test_random_requests_give_the_same_tokens_however_the_engine_runs_them(tiny_folders):
    """Eighty requests of random lengths and random sampling settings (temperature, top-k, top-p,
    repetition penalty, end of sequence on or off) through four engines - every launch from the
    interpreter, captured steps launched ahead, so few pages that requests are preempted and
    recomputed, tiny portions - give the same tokens in float32; no page and no row of seen tokens
    is lost."""
    import random
    from paged_batch_engine_b200 import SamplingParams
    cfg, _, page, _ = TINY["A"]
    folder = tiny_folders["A"]
    rnd = random.Random(5)
    V = cfg["vocab_size"]
    prompts, params = [], []
    for i in range(80):
        n = rnd.choice([1, 2, 7, 16, 17, 40, 90])
        prompts.append([rnd.randrange(V) for _ in range(n)])
        params.append(SamplingParams(max_new_tokens=rnd.choice([1, 2, 5, 20, 45]), temperature=rnd.choice([0.0, 0.7, 1.0, 1.5]),
                                     top_k=rnd.choice([0, 1, 5, 50]), top_p=rnd.choice([1.0, 0.9, 0.3]),
                                     repetition_penalty=rnd.choice([1.0, 1.0, 1.2, 0.8, 3.0]), seed=i,
                                     ignore_eos=rnd.random() < 0.7))
    outs = []
    for kw in (dict(use_cuda_graphs=False, num_pages=300), dict(num_pages=300), dict(num_pages=30, max_num_seqs=10),
               dict(num_pages=300, max_num_batched_tokens=33, prefill_chunk_cap=16)):
        eng = engine(folder, "float32", page, **kw)
        res = eng.generate(prompts, params)
        eng.runner.cache.check_invariants()
        assert eng.runner.cache.num_free_pages() == kw["num_pages"]
        assert not eng.sampler._slot_of
        outs.append([r.output_tokens for r in res])
        if kw.get("num_pages") == 30:
            assert eng.scheduler.metrics["preemptions"] > 0
    for o in outs[1:]:
        assert o == outs[0]


def test_few_pages_preempt_and_recompute_without_changing_tokens(tiny_folders):
    from paged_batch_engine_b200 import SamplingParams
    cfg, _, page, _ = TINY["A"]
    folder = tiny_folders["A"]
    prompts = prompts_for(cfg["vocab_size"], [20, 25, 30, 18], seed=7)
    sp = SamplingParams(max_new_tokens=40, ignore_eos=True)
    roomy = engine(folder, "float32", page, num_pages=64).generate(prompts, sp)
    tight_engine = engine(folder, "float32", page, num_pages=9)     # 144 tokens for 4 x (up to 70)
    tight = tight_engine.generate(prompts, sp)
    assert tight_engine.scheduler.metrics["preemptions"] > 0
    assert any(r.preemptions for r in tight)
    for a, b in zip(roomy, tight):
        assert a.output_tokens == b.output_tokens and b.finish_reason == "length"
    tight_engine.runner.cache.check_invariants()
    assert tight_engine.runner.cache.num_free_pages() == 9


def test_eos_stops_generation(tiny_folders):
    from paged_batch_engine_b200 import SamplingParams
    cfg, _, page, _ = TINY["A"]
    folder = tiny_folders["A"]
    pcfg, w = load_plain(folder)
    p = prompts_for(cfg["vocab_size"], [12], seed=11)[0]
    free = plain.greedy_generate(pcfg, w, p, 10)
    eos = free[4]
    first = free.index(eos)
    eng = engine(folder, "float32", page)
    eng.scheduler.eos = {eos}
    r = eng.generate([p], SamplingParams(max_new_tokens=10))[0]
    assert r.output_tokens == free[:first] and r.finish_reason == "stop"
    r = eng.generate([p], SamplingParams(max_new_tokens=10, ignore_eos=True))[0]
    assert r.output_tokens == free


def test_command_line(tiny_folders, tmp_path):
    cfg, _, page, _ = TINY["A"]
    folder = tiny_folders["A"]
    pcfg, w = load_plain(folder)
    prompts = prompts_for(cfg["vocab_size"], [6, 11], seed=2)
    cmd = [os.path.join(ROOT, "bin", "pbe-qwen"), folder, "--dtype", "float32", "--max-new-tokens=5",
           "--ignore-eos", "--kv-cache-blocks-per-layer=32", "--step-profile", "--request-metrics", "--final-summary"]
    for p in prompts:
        cmd += ["--prompt-ids", ",".join(map(str, p))]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    outs = [json.loads(l) for l in proc.stdout.splitlines() if l.startswith("{")]
    assert [o["output_ids"] for o in outs] == [plain.greedy_generate(pcfg, w, p, 5) for p in prompts]
    assert "steps:10" in proc.stdout and "steps/s:" in proc.stdout and "STEP_PROFILE" in proc.stdout
    metric_lines = [l for l in proc.stdout.splitlines() if l.startswith("REQUEST_METRIC ")]
    assert len(metric_lines) == 2 and all(" generated_tokens=5 " in l and " ttft_ms=" in l for l in metric_lines)
    summary = [l for l in proc.stdout.splitlines() if l.startswith("FINAL_SUMMARY ")]
    assert len(summary) == 1 and " completed_requests=2 " in summary[0] and " total_prefill_tokens=17 " in summary[0]
    # the random-weights mode writes a folder the engine can load
    cfgfile = tmp_path / "c.json"
    cfgfile.write_text(json.dumps(TINY["B"][0]))
    out = tmp_path / "rand"
    proc = subprocess.run([os.path.join(ROOT, "bin", "pbe-qwen"), "--write-random-model", str(out),
                           "--config", str(cfgfile), "--weights-seed", "4"], capture_output=True, text=True)
    assert proc.returncode == 0 and sorted(os.listdir(out)) == ["config.json", "model.safetensors"]


def test_all_layers_windowed_and_unequal_lengths_decode_together(tmp_path):
    """Every layer under a window of 300 keys, five requests of unequal length decoding in one
    captured step with key splits of 256: the request of 1,020 tokens touches two splits while
    the one of 776 touches three, so the captured step's split capacity must follow from the
    worst request, not from the longest."""
    from paged_batch_engine_b200 import SamplingParams
    from tests.helpers import TINY_C, make_model_folder
    cfg = dict(TINY_C, sliding_window=300, max_window_layers=0, max_position_embeddings=2048)
    folder = make_model_folder(tmp_path / "windowed", cfg, seed=8, sharpen=6.0)
    pcfg, w = load_plain(folder)
    prompts = prompts_for(cfg["vocab_size"], [1020, 776, 300, 50, 5], seed=13)
    sp = SamplingParams(max_new_tokens=6, ignore_eos=True)
    eng = engine(folder, "float32", 8, num_pages=400, max_num_batched_tokens=512, prefill_chunk_cap=256)
    res = eng.generate(prompts, sp)
    assert eng.runner.graphs.replays > 0
    assert all(g.window == 300 for g in eng.runner.cache.groups)
    for p, r in zip(prompts, res):
        assert r.output_tokens == plain.greedy_generate(pcfg, w, p, 6), len(p)
    eng.runner.cache.check_invariants()


def test_a_wait_that_ran_out_stops_generation_with_an_error(tiny_folders):
    """A kernel whose bounded wait ran out sets a flag on the device; the engine reads the flags
    with the sampled ids and raises instead of handing out tokens made from invalid results.
    The flag is set from the host here: nothing on the device waits, hangs or faults."""
    from paged_batch_engine_b200 import SamplingParams
    from paged_batch_engine_b200.csrc import ops as pbe_ops
    cfg, _, page, _ = TINY["D"]
    eng = engine(tiny_folders["D"], "bfloat16", page)
    prompts = prompts_for(cfg["vocab_size"], [40, 9], seed=3)
    sp = SamplingParams(max_new_tokens=6, ignore_eos=True)
    good = eng.generate(prompts, sp)
    dev = eng.device
    for when in ("prompt", "decode"):
        reqs = [eng.add_request(p, sp) for p in prompts]
        if when == "decode":
            while not all(r.outputs for r in reqs):
                eng.step()
        pbe_ops.tc5_attention_error_buffer(dev)[:1].fill_(1)
        with pytest.raises(pbe_ops.KernelError, match="bounded wait ran out.*tcgen05 attention"):
            for _ in range(4):
                eng.step()
            eng.drain()
        assert pbe_ops.tc5_error_flag(dev) == 0             # the flags were cleared when they were read
        for r in reqs:
            eng.scheduler.cancel(r)
        eng._pending = None
        eng.drain()
    # the engine is usable afterwards and gives the same tokens
    again = eng.generate(prompts, sp)
    assert [r.output_tokens for r in again] == [r.output_tokens for r in good]


def test_bfloat16_under_page_pressure_stays_plain_argmax(tiny_folders):
    """bfloat16 with so few pages that requests are preempted and recomputed (through portions
    of another size than the first time, beside other requests): every generated token is still
    the plain implementation's greedy token up to rounding, and no page is lost."""
    from paged_batch_engine_b200 import SamplingParams
    cfg, _, page, _ = TINY["A"]
    folder = tiny_folders["A"]
    pcfg, w = load_plain(folder)
    prompts = prompts_for(cfg["vocab_size"], [20, 25, 30, 18], seed=7)
    eng = engine(folder, "bfloat16", page, num_pages=9)          # 144 tokens for 4 x (up to 70)
    res = eng.generate(prompts, SamplingParams(max_new_tokens=40, ignore_eos=True))
    assert eng.scheduler.metrics["preemptions"] > 0 and any(r.preemptions for r in res)
    for p, r in zip(prompts, res):
        assert len(r.output_tokens) == 40 and r.finish_reason == "length"
        seq = p + r.output_tokens
        logits = plain.forward_logits(pcfg, w, seq[:-1])
        for i, tok in enumerate(r.output_tokens):
            row = logits[len(p) - 1 + i]
            assert row.max() - row[tok] <= 0.02 * logits.abs().max(), (len(p), i)
    eng.runner.cache.check_invariants()
    assert eng.runner.cache.num_free_pages() == 9
