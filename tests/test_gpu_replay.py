"""The engine against the plain implementation under every way of cutting and batching:
whole requests; most of a request in one step and its last 32 tokens one by one; portions
of changing size down to two tokens; up to four live requests mixed, with so few pages
that pages are used again; long decoding; the first tokens of a sequence.  In float32 and
in bfloat16, on three tiny configurations that differ in every size and option."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests import replay_util as ru
from tests.helpers import TINY, load_plain
from tests.plain import plain_qwen2 as plain

pytestmark = pytest.mark.gpu
ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))

# Stated tolerances on max |logit - plain logit| over all wanted rows.
#  float32: the engine and the plain implementation differ in summation order only.
#  bfloat16: activations between kernels are rounded to 8 bits of mantissa; the bound is
#  relative to the largest logit of the model.
TOL_F32 = 2e-5
TOL_BF16_REL = 0.02

LENGTHS = {"A": [5, 17, 33, 70], "B": [1, 9, 40, 71], "C": [3, 26, 58, 90], "D": [4, 45, 130, 301]}


def requests_for(name, vocab, extra=()):
    g = torch.Generator().manual_seed(sum(map(ord, name)))
    lens = LENGTHS[name] + list(extra)
    return {f"{name}{i}": torch.randint(0, vocab, (n,), generator=g).tolist() for i, n in enumerate(lens)}


_plain_cache = {}


def plain_logits(folder, reqs):
    cfg, w = load_plain(folder)
    out = {}
    for rid, toks in reqs.items():
        key = (folder, tuple(toks))
        if key not in _plain_cache:
            _plain_cache[key] = plain.forward_logits(cfg, w, toks)
        out[rid] = _plain_cache[key]
    return out


def make_runner(folder, dtype, page, pool_tokens, max_requests=8, **kw):
    from paged_batch_engine_b200.engine.runner import ModelRunner
    return ModelRunner.from_folder(folder, dtype=dtype, device="cuda:0", page_tokens=page,
                                   max_cache_tokens=pool_tokens, max_requests=max_requests, poison=True, **kw)


def check(got, want, dtype, label, expect_rows=None):
    """Every wanted row within the stated bound of the plain logits; and the plain
    implementation's greedy token never further below the engine's top logit than the bound
    (a missing or extra key that moves the argmax shows even under the bound)."""
    worst, where, scale = ru.max_error(got, want)
    tol = TOL_F32 if dtype == "float32" else TOL_BF16_REL * scale
    print(f"\n[replay] {label} {dtype}: max|dlogit| = {worst:.3e} at {where}, max|logit| = {scale:.3f}, tol = {tol:.3e}")
    assert worst <= tol, (label, dtype, worst, where, "first beyond tolerance:", ru.first_wrong(got, want, tol))
    n_rows = sum(len(v) for v in got.values())
    if expect_rows is None:
        expect_rows = sum(v.shape[0] for v in want.values())
    assert n_rows == expect_rows, (label, n_rows, expect_rows)
    for rid, rows in got.items():
        for pos, row in rows.items():
            top = int(want[rid][pos].argmax())
            assert float(row.max() - row[top]) <= tol, (label, rid, pos, "plain argmax is not the engine's")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_schedules_agree_with_plain(tiny_folders, name, dtype):
    cfg, _, page, _ = TINY[name]
    folder = tiny_folders[name]
    reqs = requests_for(name, cfg["vocab_size"])
    want = plain_logits(folder, reqs)
    longest = max(len(t) for t in reqs.values())
    runner = make_runner(folder, dtype, page, pool_tokens=((longest + 63) // 64) * 64)
    for label, recs in (("whole", ru.whole(reqs)), ("tail32", ru.tail_decoded(reqs)),
                        ("portions", ru.portions(reqs))):
        got = ru.run_records(runner, recs)
        assert {k: len(v) for k, v in got.items()} == {k: len(v) for k, v in reqs.items()}
        check(got, want, dtype, f"{name}/{label}")
        runner.cache.check_invariants()
        assert runner.cache.num_live_requests == 0
    # pages were handed out again and again from a pool that holds one request
    assert runner.cache.pools[0].allocations > runner.cache.pools[0].num_pages


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_mixed_batches_with_page_reuse(tiny_folders, name, dtype):
    cfg, _, page, _ = TINY[name]
    folder = tiny_folders[name]
    reqs = requests_for(name, cfg["vocab_size"], extra=(12, 47, 29, 64, 2, 65, 31, 80, 16, 55))
    want = plain_logits(folder, reqs)
    for seed in (0, 1):
        recs = ru.mixed(reqs, max_live=4, seed=seed)
        pool = ru.pool_tokens_needed(recs)        # the smallest pool the trace may be given
        runner = make_runner(folder, dtype, page, pool_tokens=pool, lifo=bool(seed))
        assert max(len(r["entries"]) for r in recs) >= 3
        assert any(len(e["tokens"]) > 1 for r in recs for e in r["entries"]) and \
            any(len(e["tokens"]) == 1 and len(r["entries"]) > 1 for r in recs for e in r["entries"])
        got = ru.run_records(runner, recs)
        check(got, want, dtype, f"{name}/mixed{seed}")
        pool0 = runner.cache.pools[0]
        assert pool0.allocations > pool0.num_pages or max(pool0.generation) >= 2   # pages were used again
        runner.cache.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_long_decoding_and_first_tokens(tiny_folders, name, dtype):
    """A request decoded one token at a time from its first token to beyond the first
    key split (256 keys) and, for C, far beyond the window; and requests of one and two
    tokens."""
    cfg, _, page, _ = TINY[name]
    folder = tiny_folders[name]
    g = torch.Generator().manual_seed(99)
    reqs = {"long": torch.randint(0, cfg["vocab_size"], (300,), generator=g).tolist(),
            "one": [7], "two": [3, 5]}
    want = plain_logits(folder, reqs)
    runner = make_runner(folder, dtype, page, pool_tokens=320 + 128)
    recs = ru.tail_decoded({"long": reqs["long"]}, tail=299) + [
        {"step": 1000, "entries": [{"id": "one", "tokens": [7], "want": [0]},
                                   {"id": "two", "tokens": [3, 5], "want": [0, 1]}], "end": ["one", "two"]}]
    got = ru.run_records(runner, recs)
    check(got, want, dtype, f"{name}/long-decode")
    if name == "C":   # the windowed group gave pages back while the full group kept them
        full_g = [i for i, s in enumerate(runner.cache.groups) if s.window is None][0]
        win_g = [i for i, s in enumerate(runner.cache.groups) if s.window is not None][0]
        assert runner.cache.pools[win_g].allocations == runner.cache.pools[full_g].allocations
        assert runner.cache.num_free_pages(win_g) == runner.cache.pools[win_g].num_pages


def test_schedules_do_not_change_float32_logits_beyond_rounding(tiny_folders):
    """Whole, portions and mixed runs of the same requests agree with each other far more
    closely than with the plain implementation's summation order."""
    cfg, _, page, _ = TINY["B"]
    reqs = requests_for("B", cfg["vocab_size"])
    runner = make_runner(tiny_folders["B"], "float32", page, pool_tokens=512)
    a = ru.run_records(runner, ru.whole(reqs))
    b = ru.run_records(runner, ru.portions(reqs))
    c = ru.run_records(runner, ru.mixed(reqs, seed=3))
    for other in (b, c):
        worst = max((a[r][p] - other[r][p]).abs().max().item() for r in a for p in a[r])
        assert worst <= 2e-5


def test_matrices_stored_in_32_bits_stay_so_in_a_bfloat16_run(tiny_folders, tmp_path):
    """A checkpoint whose output projection and LM head are stored in float32 beside bfloat16
    tensors: the bfloat16 run keeps them in float32 (true float32 products for them) and still
    agrees with the plain implementation; decoded tokens and a prompt portion both."""
    import shutil
    from safetensors.torch import load_file, save_file
    cfg, _, page, _ = TINY["B"]
    folder = str(tmp_path / "mixed_dtypes")
    shutil.copytree(tiny_folders["B"], folder)
    f = os.path.join(folder, "model.safetensors")
    w = load_file(f)
    kept = [k for k in w if k.endswith("layers.1.self_attn.o_proj.weight") or k == "lm_head.weight"]
    assert len(kept) == 2
    for k in kept:
        w[k] = w[k].float()
    save_file(w, f)
    reqs = requests_for("B", cfg["vocab_size"])
    want = plain_logits(folder, reqs)
    runner = make_runner(folder, "bfloat16", page, pool_tokens=256)
    assert runner.model.lm_head.dtype == torch.float32
    assert runner.model.blocks[1].mixer.w_o.dtype == torch.float32
    assert runner.model.blocks[0].mixer.w_o.dtype == torch.bfloat16
    for label, recs in (("whole", ru.whole(reqs)), ("tail32", ru.tail_decoded(reqs))):
        check(ru.run_records(runner, recs), want, "bfloat16", f"B/float32 matrices/{label}")


def test_trace_run_program(tiny_folders, tmp_path):
    """The program itself, as a user calls it: steps on standard input, <step>.f32 files,
    a ``done`` line after every step, exit code 0."""
    cfg, _, page, _ = TINY["A"]
    folder = tiny_folders["A"]
    reqs = requests_for("A", cfg["vocab_size"])
    want = plain_logits(folder, reqs)
    recs = ru.mixed(reqs, max_live=4, seed=5)
    for r in recs:                       # also steps that want nothing, and partial wants
        if r["step"] % 3 == 1:
            for e in r["entries"]:
                e["want"] = e["want"][-1:]
    recs[2]["entries"][0]["want"] = []
    for dtype in ("float32", "bfloat16"):
        out = tmp_path / dtype
        proc = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                               "--out", str(out), "--max-tokens", "256"],
                              input="".join(json.dumps(r) + "\n" for r in recs), capture_output=True,
                              text=True, timeout=600)
        assert proc.returncode == 0, proc.stderr[-2000:]
        assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {r['step']}" for r in recs]
        progress, worst, scale = {}, 0.0, 0.0
        for r in recs:
            n_want = sum(len(e["want"]) for e in r["entries"])
            path = out / f"{r['step']}.f32"
            if n_want == 0:
                assert not path.exists()
            else:
                rows = np.fromfile(path, dtype="<f4").reshape(n_want, cfg["vocab_size"])
                i = 0
                for e in r["entries"]:
                    base = progress.get(e["id"], 0)
                    for w in e["want"]:
                        ref = want[e["id"]][base + w]
                        worst = max(worst, float(np.abs(rows[i] - ref.numpy()).max()))
                        scale = max(scale, float(ref.abs().max()))
                        i += 1
            for e in r["entries"]:
                progress[e["id"]] = progress.get(e["id"], 0) + len(e["tokens"])
        assert worst <= (TOL_F32 if dtype == "float32" else TOL_BF16_REL * scale), (dtype, worst)
    # a pool that is too small is an error, not a wrong result
    proc = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                           "--out", str(tmp_path / "small"), "--max-tokens", "16"],
                          input=json.dumps(ru.whole(reqs)[3]) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode != 0 and "cannot hold" in proc.stderr


# ---------------------------------------------------------------- captured decode steps
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_captured_decode_steps_agree_with_plain(tiny_folders, name, dtype):
    """The step generation runs most: single-token steps replayed from a captured CUDA graph
    (fixed-layout integer buffer, padded rows, idle work items, block tables filled
    incrementally).  Last 32 tokens one by one, long decoding, and mixed batches whose
    all-decode steps are captured while their prompt portions run eagerly; once more with the
    token ids handed over on the device as a step launched ahead gets them."""
    cfg, _, page, _ = TINY[name]
    folder = tiny_folders[name]
    reqs = requests_for(name, cfg["vocab_size"], extra=(12, 47, 29, 64))
    g = torch.Generator().manual_seed(5)
    long_req = {"long": torch.randint(0, cfg["vocab_size"], (300,), generator=g).tolist()}
    want = plain_logits(folder, {**reqs, **long_req})
    from paged_batch_engine_b200.engine.replay import TraceReplayer
    runner = make_runner(folder, dtype, page, pool_tokens=1024)
    for label, recs, args in (
            ("tail32", ru.tail_decoded(reqs), {}),
            ("tail32 ids on the device", ru.tail_decoded(reqs), {"device_tokens": True}),
            ("long", ru.tail_decoded(long_req, tail=290), {}),
            ("mixed", ru.mixed(reqs, max_live=4, seed=2, prefill_frac=0.4), {}),
            ("mixed ids on the device", ru.mixed(reqs, max_live=4, seed=3, prefill_frac=0.4), {"device_tokens": True})):
        rp = TraceReplayer(runner, decode_graphs=True, **args)
        got = ru.run_records(runner, recs, replayer=rp)
        ids = {e["id"] for r in recs for e in r["entries"]}
        check(got, want, dtype, f"{name}/captured {label}", expect_rows=sum(len(want[i]) for i in ids))
        assert rp.graph_steps > 0
        runner.cache.check_invariants()
        assert runner.cache.num_live_requests == 0
    assert runner.graphs.replays > 0 and len(runner.graphs.graphs) >= 2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,count,rows", [("A", 5, 8), ("B", 20, 24), ("C", 33, 48), ("D", 3, 4), ("B", 11, 16)])
def test_captured_decode_steps_with_padding_rows(tiny_folders, name, count, rows, dtype):
    """Request counts that do not fill their captured step (5 of 8 rows, 20 of 24, 33 of 48,
    3 of 4): the padding rows write nothing, and as requests end the same requests move to
    smaller captured steps."""
    cfg, _, page, _ = TINY[name]
    folder = tiny_folders[name]
    g = torch.Generator().manual_seed(count)
    lens = [int(x) for x in torch.randint(14, 75, (count,), generator=g)]
    lens[0], lens[-1] = 90, 15
    reqs = {f"r{i}": torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for i, n in enumerate(lens)}
    want = plain_logits(folder, reqs)
    from paged_batch_engine_b200.engine.replay import TraceReplayer
    recs = ru.batch_decode(reqs, decode_tokens=12)
    runner = make_runner(folder, dtype, page, pool_tokens=ru.pool_tokens_needed(recs), max_requests=64)
    rp = TraceReplayer(runner, decode_graphs=True)
    got = ru.run_records(runner, recs, replayer=rp)
    check(got, want, dtype, f"{name}/captured {count} of {rows}")
    assert rp.graph_steps >= 12
    assert rows in {b for b, _ in runner.graphs.graphs}, sorted(runner.graphs.graphs)
    runner.cache.check_invariants()


def test_a_swapped_page_is_seen_by_the_comparison(tiny_folders):
    """The comparison with the plain implementation can fail: two requests' first pages are
    exchanged in the block tables of one step (both ids lie inside the pool and are held), in
    the eager step and in the captured one, and the logits leave the tolerance."""
    from paged_batch_engine_b200.engine import graphs as graphs_mod
    from paged_batch_engine_b200.engine.replay import TraceReplayer
    cfg, _, page, _ = TINY["A"]
    folder = tiny_folders["A"]
    reqs = requests_for("A", cfg["vocab_size"])
    two = {k: reqs[k] for k in list(reqs)[2:4]}              # 33 and 70 tokens: more than one page each
    want = plain_logits(folder, two)
    for captured in (False, True):
        runner = make_runner(folder, "float32", page, pool_tokens=256)
        recs = ru.batch_decode(two, decode_tokens=2, prefill_group=2, portion=80)
        rp = TraceReplayer(runner, decode_graphs=captured)
        for rec in recs[:-1]:
            rp.run_record(rec)
        # the last step with the two requests' first pages exchanged
        if captured:
            orig_fill = graphs_mod.DecodeStepContext.fill

            def fill(self, entries, vocab_size):
                orig_fill(self, entries, vocab_size)
                bt = self._groups[0].block_table
                a, b = bt[0, 0].clone(), bt[1, 0].clone()
                bt[0, 0], bt[1, 0] = b, a
            graphs_mod.DecodeStepContext.fill = fill
        else:
            orig_bt = runner.cache.block_table
            firsts = [orig_bt(h, 0)[0] for h in rp.handles.values()]

            def block_table(handle, group=0):
                t = orig_bt(handle, group)
                t[0] = firsts[1] if t[0] == firsts[0] else firsts[0]
                return t
            runner.cache.block_table = block_table
        try:
            logits = rp.run_record(recs[-1]).float().cpu()
        finally:
            if captured:
                graphs_mod.DecodeStepContext.fill = orig_fill
        assert rp.graph_steps == (2 if captured else 0)
        worst = max((logits[i] - want[rid][len(two[rid]) - 1]).abs().max().item() for i, rid in enumerate(two))
        assert worst > 100 * TOL_F32, (captured, worst)


# ---------------------------------------------------------------- the other ways through a step
def _switch_runs(tiny_folders, name, switch, monkeypatch):
    from paged_batch_engine_b200.csrc import native_exec, ops as pbe_ops
    from paged_batch_engine_b200.engine.replay import TraceReplayer
    if switch == "python":
        monkeypatch.setenv("PBE_EXEC", "python")
    elif switch == "mma":
        monkeypatch.setenv("PBE_ATTN", "mma")
    elif switch == "unfused":
        monkeypatch.setenv("PBE_DECODE_FUSED", "0")
    elif switch == "rows":
        monkeypatch.setenv("PBE_DECODE_TILES", "rows")
    elif switch in ("stream", "stream-python"):
        # the tcgen05 weight-streaming GEMM for every projection of every step of up to 64 rows,
        # whatever the size of the matrix (by default only large matrices take it)
        for mask in ("STREAM_MASK_FEW", "STREAM_MASK", "STREAM_MASK_MANY"):
            monkeypatch.setattr(pbe_ops, mask, 15)
        monkeypatch.setattr(pbe_ops, "STREAM_MIN_WEIGHT", 0)
        native_exec._fns.clear()
        if switch == "stream-python":
            monkeypatch.setenv("PBE_EXEC", "python")
    elif switch == "tc5gemm":
        monkeypatch.setattr(pbe_ops, "TC5_MASK", 31)
    cfg, _, page, _ = TINY[name]
    reqs = requests_for(name, cfg["vocab_size"], extra=(12, 47, 29, 64, 140))
    runner = make_runner(tiny_folders[name], "bfloat16", page, pool_tokens=1024)
    assert native_exec.enabled() == (switch not in ("python", "tc5gemm", "stream-python"))
    out = {}
    for label, recs in (("whole", ru.whole(reqs)), ("tail32", ru.tail_decoded(reqs)),
                        ("mixed", ru.mixed(reqs, max_live=4, seed=4))):
        out[label] = ru.run_records(runner, recs, replayer=TraceReplayer(runner, decode_graphs=(label == "tail32")))
    return reqs, out


@pytest.mark.parametrize("switch", ["python", "mma", "unfused", "rows", "tc5gemm", "stream", "stream-python"])
@pytest.mark.parametrize("name", ["B", "D"])
def test_every_switch_of_the_step_agrees_with_plain(tiny_folders, name, switch, monkeypatch):
    """The ways through a bfloat16 step that are not the default: every launch from the
    interpreter instead of the host library's block (PBE_EXEC=python), the mma.sync prompt
    attention (PBE_ATTN=mma), separate rope / attention / merge launches for decoded tokens
    (PBE_DECODE_FUSED=0), key tiles copied row by row (PBE_DECODE_TILES=rows), the package's
    tcgen05 GEMM for many rows (PBE_GEMM=tc5), the tcgen05 weight-streaming GEMM for every projection
    of steps of up to 64 rows (from the host library's block and from the interpreter).  Each against
    the plain implementation; the interpreter's way must equal the host library's bit for bit (same
    kernels, same order).  The launchers' table of the host library is made anew where a switch adds a
    kernel to it."""
    cfg, _, page, _ = TINY[name]
    reqs, got = _switch_runs(tiny_folders, name, switch, monkeypatch)
    want = plain_logits(tiny_folders[name], reqs)
    for label, rows in got.items():
        check(rows, want, "bfloat16", f"{name}/{switch}/{label}")
    from paged_batch_engine_b200.csrc import native_exec
    native_exec._fns.clear()
    if switch == "stream":
        # the switch took: another kernel's sums are other bits somewhere
        monkeypatch.undo()
        _, base = _switch_runs(tiny_folders, name, "default", monkeypatch)
        native_exec._fns.clear()
        assert any(not torch.equal(row, base[label][rid][pos])
                   for label in got for rid in got[label] for pos, row in got[label][rid].items())
    if switch in ("python", "stream-python"):
        monkeypatch.delenv("PBE_EXEC")
        _, native = _switch_runs(tiny_folders, name, "default" if switch == "python" else "stream", monkeypatch)
        native_exec._fns.clear()
        for label in got:
            for rid in got[label]:
                for pos, row in got[label][rid].items():
                    assert torch.equal(row, native[label][rid][pos]), (label, rid, pos)
