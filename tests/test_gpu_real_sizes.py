"""Two decoder layers at the layer sizes of Qwen2.5-7B (hidden 3584, 28 query heads on 4
key/value heads, head size 128, feed-forward 18944, vocabulary 152064, pages of 16 tokens)
against the plain implementation, in float32 and in bfloat16.

The tiny configurations cover the engine's logic; this covers the instances of the kernels
that only real sizes select: the tcgen05 prompt attention at head size 128, seven query
heads a key/value head in the decode kernels, the weight-streaming GEMM at N = 37,888 with
its SwiGLU epilogue, the LM head over 152,064 tokens, the library GEMM between 9 and a few
hundred rows, and captured decode steps at these sizes."""
import pytest
import torch

from tests import replay_util as ru
from tests.helpers import load_plain, make_model_folder
from tests.plain import plain_qwen2 as plain

pytestmark = pytest.mark.gpu

REAL = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_size=3584,
            num_hidden_layers=2, num_attention_heads=28, num_key_value_heads=4, intermediate_size=18944,
            vocab_size=152064, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
            max_position_embeddings=32768, use_sliding_window=False, hidden_act="silu", eos_token_id=151645)
PAGE = 16
# Stated bounds on max |logit - plain logit|, both relative to the largest logit; the plain
# implementation runs in float64 here, so the whole difference is the engine's.  float32: a sum
# of K float32 products carries a rounding error of about 2^-24 x sqrt(K) of its magnitude
# (8e-6 for the 18,944 terms of the down projection, 4e-6 for the 3,584 of the others), and a
# logit is reached through some ten such sums in a row: 2e-5 of the largest logit (measured
# 1.1e-5).  bfloat16: the bound of the tiny configurations.  The difference there is rounding
# noise: it is spread evenly over positions and logits (largest / root mean square = 6, the tail
# of some fifty million samples), the same through either prompt attention kernel and for
# decoded tokens, and it grows with the sharpness of attention (root mean square 1.4 % of the
# logits' with the random weights as they are, where scores already spread over several units;
# 1.9 % with queries and keys scaled by 1.5), so the weights are left as drawn.
TOL_F32_REL = 2e-5
TOL_BF16_REL = 0.02


@pytest.fixture(scope="module")
def real_model(tmp_path_factory):
    folder = make_model_folder(tmp_path_factory.mktemp("real_sizes"), REAL, seed=11, sharpen=1.0)
    g = torch.Generator().manual_seed(17)
    lens = {"main": 340, "s0": 21, "s1": 58, "s2": 45, "s3": 33, "t0": 19, "t1": 27, "t2": 16, "t3": 30, "t4": 24,
            "t5": 18}
    reqs = {k: torch.randint(0, REAL["vocab_size"], (n,), generator=g).tolist() for k, n in lens.items()}
    cfg, w = load_plain(folder)
    with torch.no_grad():
        want = {k: plain.forward_logits(cfg, w, t, dtype=torch.float64).float() for k, t in reqs.items()}
    del w
    return folder, reqs, want


def _check(got, want, dtype, label):
    worst, where, scale = ru.max_error(got, want)
    tol = (TOL_F32_REL if dtype == "float32" else TOL_BF16_REL) * scale
    print(f"\n[real sizes] {label} {dtype}: max|dlogit| = {worst:.3e} at {where}, max|logit| = {scale:.3f}, "
          f"tol = {tol:.3e}")
    assert worst <= tol, (label, dtype, worst, where, ru.first_wrong(got, want, tol))
    for rid, rows in got.items():
        for pos, row in rows.items():
            top = int(want[rid][pos].argmax())
            assert float(row.max() - row[top]) <= tol, (label, rid, pos)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layers_of_real_size_agree_with_plain(real_model, dtype):
    from paged_batch_engine_b200.engine.replay import TraceReplayer
    from paged_batch_engine_b200.engine.runner import ModelRunner
    folder, reqs, want = real_model
    runner = ModelRunner.from_folder(folder, dtype=dtype, device="cuda:0", page_tokens=PAGE,
                                     max_cache_tokens=2048, max_requests=16, poison=True)
    main = {"main": reqs["main"]}
    # whole; in portions of changing size with the last 40 tokens one by one, eagerly; the same
    # with the single tokens through captured steps
    got = ru.run_records(runner, ru.whole(main))
    assert len(got["main"]) == 340
    _check(got, want, dtype, "whole")
    recs = ru.portions({"main": reqs["main"][:300]}, sizes=(128, 2, 97, 64, 9))
    recs[-1]["end"] = []
    recs += [{"step": 100 + i, "entries": [{"id": "main", "tokens": [reqs["main"][300 + i]], "want": [0]}],
              "end": ["main"] if i == 39 else []} for i in range(40)]
    for captured in (False, True):
        rp = TraceReplayer(runner, decode_graphs=captured)
        got = ru.run_records(runner, recs, replayer=rp)
        assert len(got["main"]) == 340 and rp.graph_steps == (40 if captured else 0)
        _check(got, want, dtype, "portions + 40 decoded" + (" (captured)" if captured else ""))
    # five requests decoding together (five rows in a captured step of eight)
    five = {k: reqs[k] for k in ("main", "s0", "s1", "s2", "s3")}
    recs = ru.batch_decode(five, decode_tokens=10, prefill_group=3, portion=200)
    rp = TraceReplayer(runner, decode_graphs=True, device_tokens=True)
    got = ru.run_records(runner, recs, replayer=rp)
    assert rp.graph_steps == 10 and 8 in {b for b, _ in runner.graphs.graphs}
    _check(got, want, dtype, "five requests, captured")
    # eleven together, eagerly and captured (a step of sixteen rows): in bfloat16 the gate/up and
    # down projections of such a step are the tcgen05 weight-streaming kernel's
    for captured in (False, True):
        recs = ru.batch_decode(reqs, decode_tokens=6, prefill_group=4, portion=200)
        rp = TraceReplayer(runner, decode_graphs=captured, device_tokens=captured)
        got = ru.run_records(runner, recs, replayer=rp)
        assert not captured or (rp.graph_steps == 6 and 16 in {b for b, _ in runner.graphs.graphs})
        _check(got, want, dtype, "eleven requests" + (", captured" if captured else ""))
    runner.cache.check_invariants()
    assert runner.cache.num_live_requests == 0
