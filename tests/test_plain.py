"""The plain implementation itself (no GPU): against the reference's own Python model on a
committed tiny random model, and its parts against hand-made cases."""
import math
import os

import pytest
import torch

from tests.plain import plain_qwen2 as plain

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_tiny.safetensors")


def test_plain_matches_reference_python_model():
    from safetensors.torch import load_file
    g = load_file(GOLDEN)
    tokens = g.pop("tokens").tolist()
    want = g.pop("logits")
    cfg = dict(hidden_size=32, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
               intermediate_size=48, vocab_size=61, rms_norm_eps=1e-6, rope_theta=10000.0,
               tie_word_embeddings=True)
    got = plain.forward_logits(cfg, g, tokens, rope=plain.rope_interleaved)
    assert got.shape == want.shape == (19, 61)
    assert (got - want).abs().max().item() < 2e-5 * max(1.0, want.abs().max().item())
    assert want.abs().max().item() > 0.5            # the model is not degenerate
    # the engine's pairing gives different logits: the anchor would notice a mix-up
    other = plain.forward_logits(cfg, g, tokens, rope=plain.rope_rotate_half)
    assert (other - want).abs().max().item() > 1e-2


def test_rmsnorm_by_hand():
    x = torch.tensor([[3.0, 4.0]])
    y = plain.rmsnorm(x, torch.tensor([2.0, 0.5]), eps=0.0)
    s = 1.0 / math.sqrt(12.5)
    assert torch.allclose(y, torch.tensor([[6.0 * s, 2.0 * s]]))


def test_rope_rotate_half_by_hand():
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0]]])       # one token, one head, head_dim 4
    y = plain.rope_rotate_half(x, torch.tensor([3]), theta=100.0)
    f = [1.0, 100.0 ** (-0.5)]
    exp = [1 * math.cos(3 * f[0]) - 3 * math.sin(3 * f[0]), 2 * math.cos(3 * f[1]) - 4 * math.sin(3 * f[1]),
           3 * math.cos(3 * f[0]) + 1 * math.sin(3 * f[0]), 4 * math.cos(3 * f[1]) + 2 * math.sin(3 * f[1])]
    assert torch.allclose(y.flatten(), torch.tensor(exp), atol=1e-6)
    assert torch.equal(plain.rope_rotate_half(x, torch.tensor([0]), 100.0), x)


def test_attention_is_causal_grouped_and_windowed():
    torch.manual_seed(0)
    T, H, KV, hd = 7, 4, 2, 8
    q, k, v = torch.randn(T, H, hd), torch.randn(T, KV, hd), torch.randn(T, KV, hd)
    o = plain.causal_attention(q, k, v, hd ** -0.5)
    assert torch.allclose(o[0, 1], v[0, 0]) and torch.allclose(o[0, 3], v[0, 1])   # first row sees itself
    k2, v2 = k.clone(), v.clone()
    k2[5:], v2[5:] = 9.0, -9.0                       # the future does not matter
    assert torch.allclose(plain.causal_attention(q, k2, v2, hd ** -0.5)[:5], o[:5])
    ow = plain.causal_attention(q, k, v, hd ** -0.5, window=3)
    assert torch.allclose(ow[:3], o[:3]) and not torch.allclose(ow[3:], o[3:])
    k3 = k.clone()
    k3[0] += 50.0 * q[6, 0, :].sign().mean()         # key 0 is outside row 6's window of 3
    assert torch.allclose(plain.causal_attention(q, k3, v, hd ** -0.5, window=3)[6], ow[6])


def test_swiglu_and_uniform():
    g, u = torch.tensor([0.0, 2.0]), torch.tensor([5.0, 3.0])
    assert torch.allclose(plain.swiglu(g, u), torch.tensor([0.0, 2.0 / (1 + math.exp(-2.0)) * 3.0]))
    # fixed points of the counter-based generator (SplitMix64 of seed + phi * (counter + 1))
    u0 = plain.request_sample_uniform(0xC0FFEE, 0)
    assert 0.0 <= u0 < 1.0 and u0 == plain.request_sample_uniform(0xC0FFEE, 0)
    assert u0 != plain.request_sample_uniform(0xC0FFEE, 1) != plain.request_sample_uniform(0xC0FFEF, 1)
    vals = [plain.request_sample_uniform(7, c) for c in range(2000)]
    assert 0.45 < sum(vals) / len(vals) < 0.55


def test_sampler_rules():
    logits = [0.1, 2.0, 2.0, -1.0, 1.5]
    assert plain.sample_row(logits) == 1                                   # ties: lowest id
    assert plain.sample_row(logits, temperature=0.7, top_k=1, uniform=0.99) == 1
    # top_k=3 keeps tokens 1, 2, 4; with u near 1 the last of them in probability order
    assert plain.sample_row(logits, temperature=1.0, top_k=3, uniform=0.999) == 4
    assert plain.sample_row(logits, temperature=1.0, top_k=3, uniform=0.0) == 1
    # top_p small: only the first candidate survives
    assert plain.sample_row(logits, temperature=1.0, top_p=0.2, uniform=0.9) == 1
    # repetition penalty pushes seen tokens down (positive logits are divided)
    assert plain.sample_row(logits, temperature=1e-3, repetition_penalty=4.0, seen_tokens=[1, 2], uniform=0.5) == 4
    lo, hi = plain.sample_cdf_interval(logits, 2, 1.0, top_k=3)
    assert 0 < lo < hi < 1


def test_rotary_pairing_matches_the_reference_cpp_kernel():
    """The reference's own C++ CPU rotary kernel in its Qwen2 branch (compiled unmodified by
    tests/golden/make_reference_rope_golden.py) against the plain implementation: the pairing
    (i, i + head_size/2), the direction of the rotation and every pair's frequency with
    theta = 1e6, for query and key heads, at positions up to 4,095."""
    from safetensors.torch import load_file
    g = load_file(os.path.join(os.path.dirname(__file__), "golden", "reference_rope.safetensors"))
    for tag in ("a", "b", "c"):
        head_size, heads, kv_heads = g[f"{tag}.shape"].tolist()
        pos = g[f"{tag}.positions"].long()
        for name, n in (("q", heads), ("k", kv_heads)):
            x = g[f"{tag}.{name}"].view(len(pos), n, head_size)
            want = g[f"{tag}.{name}_rotated"].view(len(pos), n, head_size)
            got = plain.rope_rotate_half(x, pos, theta=1000000.0)
            # both take sine and cosine of the same float32 angle: a few units in the last place
            assert (got - want).abs().max().item() <= 2e-6, (tag, name)
            small = pos <= 64
            assert not torch.allclose(got[1:], x[1:], atol=1e-3)                       # it did rotate
            wrong = plain.rope_interleaved(x, pos, theta=1000000.0)
            assert (wrong[small][1:] - want[small][1:]).abs().max().item() > 1e-2       # a mix-up shows
