"""Each part of a layer alone against the plain functions, and the framework's openness:
a toy mixer with state of its own, a toy architecture whose run order names a block twice
and lets a layer read another layer's cache, all defined here and registered without a
change to the package's files."""
import math
from dataclasses import dataclass
from typing import Optional

import pytest
import torch

from tests.plain import plain_qwen2 as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ctx(manager, entries, work_keys):
    from paged_batch_engine_b200.engine.batch import StepContext
    return StepContext(manager, entries, torch.device(DEV), work_keys)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_and_feed_forward_parts(dtype):
    from paged_batch_engine_b200.config import PartSpec
    from paged_batch_engine_b200.parts import build_part
    torch.manual_seed(0)
    d, inter, T = 88, 208, 9
    norm = build_part("norm", PartSpec("rmsnorm", dict(size=d, eps=3e-6)), dtype, DEV)
    assert [p.name for p in norm.param_specs("x.")] == ["x.weight"]
    gain = 1 + 0.1 * torch.randn(d)
    norm.load({"x.weight": gain.to(DEV)}, "x.")
    res = torch.randn(T, d)
    r = res.clone().to(DEV)
    y = norm.add_norm(r, None)
    tol = 1e-5 if dtype == torch.float32 else 2 ** -7
    assert (y.float().cpu() - plain.rmsnorm(res, gain, 3e-6)).abs().max() <= tol * 4

    ffn = build_part("feed_forward", PartSpec("swiglu", dict(hidden_size=d, intermediate_size=inter)), dtype, DEV)
    w = {"m.gate_proj.weight": torch.randn(inter, d) * 0.1, "m.up_proj.weight": torch.randn(inter, d) * 0.1,
         "m.down_proj.weight": torch.randn(d, inter) * 0.1}
    w = {k: v.to(dtype) for k, v in w.items()}
    assert sorted(p.name for p in ffn.param_specs("m.")) == sorted(w)
    ffn.load({k: v.to(DEV) for k, v in w.items()}, "m.")
    x = torch.randn(T, d).to(dtype)
    got = ffn.forward(x.to(DEV), None).float().cpu()
    want = plain.feed_forward(x.float(), {k: v.float() for k, v in w.items()}, "m.")
    assert (got - want).abs().max() <= (1e-5 if dtype == torch.float32 else 0.03) * max(1.0, want.abs().max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 10])
def test_attention_part_whole_and_in_portions(dtype, window):
    from paged_batch_engine_b200.cache import CacheManager, KVGroupSpec
    from paged_batch_engine_b200.cache.storage import CacheStorage
    from paged_batch_engine_b200.config import PartSpec
    from paged_batch_engine_b200.engine.batch import StepEntry
    from paged_batch_engine_b200.parts import build_part
    torch.manual_seed(1)
    d, H, KV, hd, T, P = 72, 6, 2, 32, 45, 8
    spec = PartSpec("attention", dict(hidden_size=d, num_heads=H, num_kv_heads=KV, head_dim=hd,
                                      window=window, qkv_bias=True, o_bias=False,
                                      position=PartSpec("rope", dict(theta=777.0, head_dim=hd))))
    attn = build_part("mixer", spec, dtype, DEV)
    cfg = dict(num_attention_heads=H, num_key_value_heads=KV, head_dim=hd, hidden_size=d, rope_theta=777.0)
    w = {}
    for p in attn.param_specs("a."):
        w[p.name] = (torch.randn(p.shape) * (0.4 if "q_proj.w" in p.name or "k_proj.w" in p.name else 0.15)).to(
            dtype if len(p.shape) > 1 else torch.float32)
    attn.load({k: v.to(DEV) for k, v in w.items()}, "a.")
    x = torch.randn(T, d).to(dtype)
    want = plain.attention_block(x.float(), torch.arange(T), {k: v.float() for k, v in w.items()}, "a.", cfg, window)
    storage = CacheStorage([attn.cache_need()], P, 16, 4, dtype, torch.device(DEV), poison=True)
    keys = [(0,) + k for k in attn.work_keys()]
    for cuts in ([T], [7, 2, 16, 1, 19]):
        h = storage.manager.add_request()
        outs, i = [], 0
        for n in cuts:
            assert storage.manager.reserve(h, n)
            ctx = _ctx(storage.manager, [StepEntry(h, [0] * n)], keys)
            outs.append(attn.forward(x[i:i + n].to(DEV).contiguous(), ctx, storage.layer(0)).float().cpu())
            storage.manager.commit(h, n)
            i += n
        storage.manager.free(h)
        got = torch.cat(outs)
        tol = 2e-5 if dtype == torch.float32 else 0.03
        assert (got - want).abs().max() <= tol * max(1.0, want.abs().max()), cuts


def test_position_encoding_part():
    from paged_batch_engine_b200.config import PartSpec
    from paged_batch_engine_b200.parts import build_part
    rope = build_part("position", PartSpec("rope", dict(theta=50000.0, head_dim=48, rotary_dim=32)), torch.float32, DEV)
    inv, rot, inter = rope.kernel_args()
    assert rot == 32 and inter is False and inv.dtype == torch.float32
    assert torch.equal(inv.cpu(), plain.rope_inv_freq(32, 50000.0))
    none = build_part("position", PartSpec("none"), torch.float32, DEV)
    assert none.kernel_args() == (None, 0, False)
    with pytest.raises(ValueError):
        build_part("position", PartSpec("rope", dict(theta=1e4, head_dim=16, rotary_dim=18)), torch.float32, DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_block_alone(dtype):
    """A pre-norm block built from its BlockSpec, stepped whole and in two portions, against
    the plain functions put together the same way."""
    from paged_batch_engine_b200.cache.storage import CacheStorage
    from paged_batch_engine_b200.config import BlockSpec, PartSpec
    from paged_batch_engine_b200.engine.batch import StepEntry
    from paged_batch_engine_b200.parts import build_block
    torch.manual_seed(3)
    d, H, KV, hd, inter, T, P, eps = 56, 4, 2, 16, 104, 29, 8, 2e-5
    norm = PartSpec("rmsnorm", dict(size=d, eps=eps))
    spec = BlockSpec("prenorm",
                     PartSpec("attention", dict(hidden_size=d, num_heads=H, num_kv_heads=KV, head_dim=hd,
                                                position=PartSpec("rope", dict(theta=900.0, head_dim=hd)))),
                     PartSpec("swiglu", dict(hidden_size=d, intermediate_size=inter)), norm, norm, "blk.",
                     dict(mixer="att.", feed_forward="ff.", norm_mixer="n1.", norm_feed_forward="n2."))
    block = build_block(spec, dtype, torch.device(DEV))
    w = {}
    for p in block.param_specs():
        t = torch.randn(p.shape) * (0.5 if "q_proj.w" in p.name or "k_proj.w" in p.name else 0.2)
        if p.name.endswith("n1.weight") or p.name.endswith("n2.weight"):
            t = 1 + 0.1 * torch.randn(p.shape)
        w[p.name] = t.to(dtype if len(p.shape) > 1 else torch.float32)
    block.load({k: v.to(DEV) for k, v in w.items()})
    wf = {k: v.float() for k, v in w.items()}
    x = torch.randn(T, d)
    cfg = dict(num_attention_heads=H, num_key_value_heads=KV, head_dim=hd, hidden_size=d, rope_theta=900.0)
    h = plain.rmsnorm(x, wf["blk.n1.weight"], eps)
    x1 = x + plain.attention_block(h, torch.arange(T), wf, "blk.att.", cfg, None)
    want = x1 + plain.feed_forward(plain.rmsnorm(x1, wf["blk.n2.weight"], eps), wf, "blk.ff.")
    storage = CacheStorage([block.mixer.cache_need()], P, 8, 2, dtype, torch.device(DEV), poison=True)
    keys = [(0,) + k for k in block.mixer.work_keys()]
    for cuts in ([T], [11, 18]):
        hnd = storage.manager.add_request()
        outs, i = [], 0
        for n in cuts:
            assert storage.manager.reserve(hnd, n)
            ctx = _ctx(storage.manager, [StepEntry(hnd, [0] * n)], keys)
            res = x[i:i + n].clone().to(DEV)
            res, delta = block.forward(res, None, ctx, storage.layer(0))
            outs.append((res + delta.float()).cpu())
            storage.manager.commit(hnd, n)
            i += n
        storage.manager.free(hnd)
        got = torch.cat(outs)
        tol = 3e-5 if dtype == torch.float32 else 0.04
        assert (got - want).abs().max() <= tol * max(1.0, want.abs().max()), cuts


# ------------------------------------------------------------------ toy parts, defined in the test
def _toy_decay():
    return 0.75


def make_toy_mixer_class():
    from paged_batch_engine_b200.parts import Mixer, StateNeed
    from paged_batch_engine_b200.weights import ParamSpec

    class ToyStateMixer(Mixer):
        """y_t = s_t with s_t = decay * s_{t-1} + x_t * w: a mixer with a fixed-size state per
        request, no pages.  The state lives in the request's slot between steps."""

        def __init__(self, hidden_size, dtype, device, decay=0.5):
            self.d, self.decay, self.dtype, self.device = hidden_size, decay, dtype, device
            self.w = None

        def cache_need(self):
            return StateNeed((self.d,), torch.float32)

        def param_specs(self, prefix):
            return [ParamSpec(prefix + "mix", (self.d,))]

        def load(self, tensors, prefix):
            self.w = tensors.pop(prefix + "mix").float()

        def forward(self, x, ctx, cache):
            y = torch.empty_like(x)
            for r in range(ctx.num_requests):
                lo, n = int(ctx.q_start_host[r]), int(ctx.q_len_host[r])
                slot = int(ctx.state_slots_host[r])
                s = cache.state[slot]
                if ctx.context_before_host[r] == 0:
                    s.zero_()                      # a new request starts from an empty state
                for t in range(lo, lo + n):
                    s.mul_(self.decay).add_(x[t].float() * self.w)
                    y[t] = s.to(x.dtype)
            return y

    return ToyStateMixer


def plain_toy_model(cfg, w, tokens):
    """The toy architecture, whole sequence, plain: see ToyConfig.model_spec below."""
    x = plain.embedding(tokens, w["emb"])
    pos = torch.arange(len(tokens))
    acfg = dict(num_attention_heads=cfg["heads"], num_key_value_heads=cfg["kv"], head_dim=cfg["hd"],
                hidden_size=cfg["d"], rope_theta=cfg["theta"])

    def attn_layer(x, p, kv_from=None):
        h = plain.rmsnorm(x, w[p + "n1.weight"], cfg["eps"])
        ww = dict(w)
        if kv_from is not None:        # reads the keys and values another layer computed
            T, H, KV, hd = len(tokens), cfg["heads"], cfg["kv"], cfg["hd"]
            q = plain.linear(h, w[p + "at.q_proj.weight"], w[p + "at.q_proj.bias"]).view(T, H, hd)
            q = plain.rope_rotate_half(q, pos, cfg["theta"])
            o = plain.causal_attention(q, kv_from[0], kv_from[1], hd ** -0.5)
            a = plain.linear(o.reshape(T, H * hd), w[p + "at.o_proj.weight"])
            kv = kv_from
        else:
            T, H, KV, hd = len(tokens), cfg["heads"], cfg["kv"], cfg["hd"]
            k = plain.rope_rotate_half(plain.linear(h, w[p + "at.k_proj.weight"], w[p + "at.k_proj.bias"]).view(T, KV, hd), pos, cfg["theta"])
            v = plain.linear(h, w[p + "at.v_proj.weight"], w[p + "at.v_proj.bias"]).view(T, KV, hd)
            a = plain.attention_block(h, pos, ww, p + "at.", acfg, None)
            kv = (k, v)
        x = x + a
        f = plain.rmsnorm(x, w[p + "n2.weight"], cfg["eps"])
        return x + plain.feed_forward(f, w, p + "ff."), kv

    def toy_layer(x, p):
        h = plain.rmsnorm(x, w[p + "n1.weight"], cfg["eps"])
        s = torch.zeros(cfg["d"])
        out = []
        for t in range(len(tokens)):
            s = _toy_decay() * s + h[t] * w[p + "tm.mix"]
            out.append(s.clone())
        x = x + torch.stack(out)
        f = plain.rmsnorm(x, w[p + "n2.weight"], cfg["eps"])
        return x + plain.feed_forward(f, w, p + "ff.")

    x, kv0 = attn_layer(x, "L0.")            # block 0, cache layer 0
    x = toy_layer(x, "L1.")                  # block 1, state in cache layer 1
    x, _ = attn_layer(x, "L2.", kv_from=kv0)  # block 2 reads cache layer 0, writes nothing
    x = toy_layer(x, "L1.")                  # block 1 again, with a state of its own (cache layer 2)
    x = plain.rmsnorm(x, w["fn.weight"], cfg["eps"])
    return plain.linear(x, w["head"])


def test_toy_architecture_registers_builds_and_steps():
    from paged_batch_engine_b200.config import (BlockSpec, ModelSpec, PartSpec, RunStep, load_config,
                                                register_architecture)
    from paged_batch_engine_b200.engine.batch import StepEntry
    from paged_batch_engine_b200.engine.runner import ModelRunner, build_model
    from paged_batch_engine_b200.parts import register_part
    from paged_batch_engine_b200.weights import random_state_dict

    register_part("mixer", "toy_state", make_toy_mixer_class(), replace=True)

    @dataclass
    class ToyConfig:
        d: int = 40
        heads: int = 4
        kv: int = 2
        hd: int = 16
        inter: int = 56
        vocab: int = 97
        eps: float = 2e-5
        theta: float = 300.0

        @classmethod
        def from_dict(cls, d):
            return cls(**{k: v for k, v in d.items() if k in cls.__dataclass_fields__})

        def model_spec(self):
            norm = PartSpec("rmsnorm", dict(size=self.d, eps=self.eps))
            ffn = PartSpec("swiglu", dict(hidden_size=self.d, intermediate_size=self.inter))
            attn = PartSpec("attention", dict(hidden_size=self.d, num_heads=self.heads, num_kv_heads=self.kv,
                                              head_dim=self.hd, position=PartSpec("rope", dict(theta=self.theta, head_dim=self.hd))))
            toy = PartSpec("toy_state", dict(hidden_size=self.d, decay=_toy_decay()))
            names = dict(norm_mixer="n1.", norm_feed_forward="n2.", feed_forward="ff.")
            blocks = (BlockSpec("prenorm", attn, ffn, norm, norm, "L0.", dict(names, mixer="at.")),
                      BlockSpec("prenorm", toy, ffn, norm, norm, "L1.", dict(names, mixer="tm.")),
                      BlockSpec("prenorm", attn, ffn, norm, norm, "L2.", dict(names, mixer="at.")))
            run = (RunStep(0, 0), RunStep(1, 1), RunStep(2, 0, writes_cache=False), RunStep(1, 2))
            return ModelSpec("ToyForCausalLM", self.d, self.vocab, blocks, run, norm, "emb", "fn.", "head", 512)

    register_architecture("ToyForCausalLM", ToyConfig, replace=True)
    arch, cfg = load_config({"architectures": ["ToyForCausalLM"], "vocab": 97})
    assert arch.name == "ToyForCausalLM"
    for dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 0.05)):
        model = build_model(cfg, dtype, torch.device(DEV))
        assert [type(n).__name__ for n in model.cache_needs] == ["KVNeed", "StateNeed", "StateNeed"]
        sd = random_state_dict(model.param_specs(), seed=3, dtype=torch.float32)
        for k in sd:
            if "q_proj.weight" in k or "k_proj.weight" in k:
                sd[k] = sd[k] * 10
            if k.endswith("mix"):
                sd[k] = torch.linspace(0.5, 1.5, 40)
        if dtype == torch.bfloat16:
            sd = {k: (v.to(torch.bfloat16) if v.dim() > 1 else v) for k, v in sd.items()}
        model.build_kernels()
        model.load({k: v.to(DEV) for k, v in sd.items()})
        runner = ModelRunner(model, page_tokens=8, num_pages=12, max_requests=3)
        toks = {"a": torch.randint(0, 97, (37,), generator=torch.Generator().manual_seed(1)).tolist(),
                "b": torch.randint(0, 97, (20,), generator=torch.Generator().manual_seed(2)).tolist()}
        want = {k: plain_toy_model(cfg.__dict__, {n: t.float() for n, t in sd.items()}, v) for k, v in toks.items()}
        # whole, then interleaved portions of both requests with single tokens at the end
        for plan in ([("a", 37)], [("b", 20)],
                     [("a", 5), ("b", 3), ("a", 2), ("b", 16), ("a", 29), ("b", 1), ("a", 1)]):
            handles, done, got = {}, {}, {}
            i = 0
            while i < len(plan):
                batch = [plan[i]]
                if i + 1 < len(plan) and plan[i + 1][0] != plan[i][0] and len(plan) > 2:
                    batch.append(plan[i + 1])
                i += len(batch)
                entries = []
                for rid, n in batch:
                    if rid not in handles:
                        handles[rid] = runner.cache.add_request()
                        done[rid] = 0
                    assert runner.cache.reserve(handles[rid], n)
                    entries.append(StepEntry(handles[rid], toks[rid][done[rid]:done[rid] + n], list(range(n))))
                logits = runner.step(entries).float().cpu()
                j = 0
                for rid, n in batch:
                    got.setdefault(rid, []).append(logits[j:j + n])
                    j += n
                    done[rid] += n
            for rid in handles:
                runner.cache.free(handles[rid])
                out = torch.cat(got[rid])
                assert out.shape == want[rid][:len(out)].shape
                err = (out - want[rid][:len(out)]).abs().max().item()
                assert err <= tol * max(1.0, want[rid].abs().max().item()), (dtype, plan, rid, err)


# ------------------------------------------------------------------ a toy feed-forward with routing, a toy position encoding
def make_toy_routed_ffn_class():
    from paged_batch_engine_b200.parts import FeedForward
    from paged_batch_engine_b200.weights import ParamSpec

    class ToyRoutedFFN(FeedForward):
        """Router logits x R^T in float32, softmax over the ``top_k`` largest, and the weighted sum
        of those experts' relu(x A_e^T) B_e^T: a feed-forward whose experts are chosen per token."""

        def __init__(self, hidden_size, experts, expert_size, top_k, dtype, device):
            self.d, self.E, self.m, self.k, self.dtype = hidden_size, experts, expert_size, top_k, dtype

        def param_specs(self, prefix):
            return [ParamSpec(prefix + "router", (self.E, self.d)),
                    ParamSpec(prefix + "a", (self.E * self.m, self.d)), ParamSpec(prefix + "b", (self.E * self.d, self.m))]

        def load(self, tensors, prefix):
            self.router = tensors.pop(prefix + "router").float()
            self.a = tensors.pop(prefix + "a").float().view(self.E, self.m, self.d)
            self.b = tensors.pop(prefix + "b").float().view(self.E, self.d, self.m)

        def forward(self, x, ctx):
            xf = x.float()
            top, idx = (xf @ self.router.t()).topk(self.k, dim=-1)
            gate = torch.softmax(top, dim=-1)
            y = torch.zeros_like(xf)
            for e in range(self.E):
                rows, slot = (idx == e).nonzero(as_tuple=True)
                if len(rows):
                    h = torch.relu(xf[rows] @ self.a[e].t()) @ self.b[e].t()
                    y.index_add_(0, rows, h * gate[rows, slot].unsqueeze(1))
            return y.to(self.dtype)

    return ToyRoutedFFN


def make_toy_position_class():
    from paged_batch_engine_b200.parts import PositionEncoding
    from paged_batch_engine_b200.weights import ParamSpec

    class ToyTablePosition(PositionEncoding):
        """q and k get a learned vector of their position (modulo ``period``) added: a position
        encoding with a tensor of its own and code of its own."""
        applies_itself = True

        def __init__(self, head_dim, period, dtype, device):
            self.hd, self.period = head_dim, period

        def param_specs(self, prefix):
            return [ParamSpec(prefix + "table", (self.period, self.hd))]

        def load(self, tensors, prefix):
            self.table = tensors.pop(prefix + "table").float()

        def apply(self, q, k, positions):
            add = self.table[(positions % self.period).long()].unsqueeze(1)
            return q + add, k + add

    return ToyTablePosition


def plain_toy_routed_ffn(f, w, p, E, top_k):
    """Per token: the top_k router logits, their softmax, the weighted experts."""
    out = []
    for t in range(f.shape[0]):
        logits = w[p + "router"] @ f[t]
        order = sorted(range(E), key=lambda e: -logits[e].item())[:top_k]
        gate = torch.softmax(torch.stack([logits[e] for e in order]), 0)
        y = torch.zeros_like(f[t])
        for g, e in zip(gate, order):
            a = w[p + "a"].view(E, -1, f.shape[1])[e]
            b = w[p + "b"].view(E, f.shape[1], -1)[e]
            y = y + g * (b @ torch.relu(a @ f[t]))
        out.append(y)
    return torch.stack(out)


def plain_toy_model_2(c, w, tokens):
    """Block 0: attention with the table position encoding, routed feed-forward; block 1:
    attention with rotary encoding and a window, SwiGLU."""
    T, H, KV, hd = len(tokens), c["heads"], c["kv"], c["hd"]
    pos = torch.arange(T)
    x = plain.embedding(tokens, w["emb"])
    h = plain.rmsnorm(x, w["A.n1.weight"], c["eps"])
    q = plain.linear(h, w["A.at.q_proj.weight"], w["A.at.q_proj.bias"]).view(T, H, hd)
    k = plain.linear(h, w["A.at.k_proj.weight"], w["A.at.k_proj.bias"]).view(T, KV, hd)
    v = plain.linear(h, w["A.at.v_proj.weight"], w["A.at.v_proj.bias"]).view(T, KV, hd)
    add = w["A.at.position.table"][pos % c["period"]].unsqueeze(1)
    o = plain.causal_attention(q + add, k + add, v, hd ** -0.5)
    x = x + plain.linear(o.reshape(T, H * hd), w["A.at.o_proj.weight"])
    f = plain.rmsnorm(x, w["A.n2.weight"], c["eps"])
    x = x + plain_toy_routed_ffn(f, w, "A.ff.", c["experts"], c["top_k"])
    acfg = dict(num_attention_heads=H, num_key_value_heads=KV, head_dim=hd, hidden_size=c["d"], rope_theta=c["theta"])
    h = plain.rmsnorm(x, w["B.n1.weight"], c["eps"])
    x = x + plain.attention_block(h, pos, w, "B.at.", acfg, c["window"])
    f = plain.rmsnorm(x, w["B.n2.weight"], c["eps"])
    x = x + plain.feed_forward(f, w, "B.ff.")
    return plain.linear(plain.rmsnorm(x, w["fn.weight"], c["eps"]), w["head"])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_toy_routed_feed_forward_and_toy_position_encoding(dtype):
    """A feed-forward with routing and a position encoding with code and a tensor of its own, both
    defined here, are registered, chosen layer by layer beside the package's own parts, and
    stepped whole, in portions and token by token, with no change to the package."""
    from paged_batch_engine_b200.config import (BlockSpec, ModelSpec, PartSpec, RunStep, load_config,
                                                register_architecture)
    from paged_batch_engine_b200.engine.batch import StepEntry
    from paged_batch_engine_b200.engine.runner import ModelRunner, build_model
    from paged_batch_engine_b200.parts import register_part
    from paged_batch_engine_b200.weights import random_state_dict

    register_part("feed_forward", "toy_routed", make_toy_routed_ffn_class(), replace=True)
    register_part("position", "toy_table", make_toy_position_class(), replace=True)

    @dataclass
    class Toy2Config:
        d: int = 48
        heads: int = 6
        kv: int = 3
        hd: int = 32
        inter: int = 72
        vocab: int = 101
        eps: float = 3e-6
        theta: float = 500.0
        period: int = 7
        experts: int = 3
        expert_size: int = 20
        top_k: int = 1
        window: int = 24

        @classmethod
        def from_dict(cls, d):
            return cls(**{k: v for k, v in d.items() if k in cls.__dataclass_fields__})

        def model_spec(self):
            norm = PartSpec("rmsnorm", dict(size=self.d, eps=self.eps))
            att = dict(hidden_size=self.d, num_heads=self.heads, num_kv_heads=self.kv, head_dim=self.hd)
            att_a = PartSpec("attention", dict(att, position=PartSpec("toy_table", dict(head_dim=self.hd, period=self.period))))
            att_b = PartSpec("attention", dict(att, window=self.window,
                                               position=PartSpec("rope", dict(theta=self.theta, head_dim=self.hd))))
            routed = PartSpec("toy_routed", dict(hidden_size=self.d, experts=self.experts, expert_size=self.expert_size,
                                                 top_k=self.top_k))
            dense = PartSpec("swiglu", dict(hidden_size=self.d, intermediate_size=self.inter))
            names = dict(norm_mixer="n1.", norm_feed_forward="n2.", feed_forward="ff.", mixer="at.")
            blocks = (BlockSpec("prenorm", att_a, routed, norm, norm, "A.", names),
                      BlockSpec("prenorm", att_b, dense, norm, norm, "B.", names))
            return ModelSpec("Toy2ForCausalLM", self.d, self.vocab, blocks, (RunStep(0, 0), RunStep(1, 1)), norm,
                             "emb", "fn.", "head", 512)

    register_architecture("Toy2ForCausalLM", Toy2Config, replace=True)
    # one expert a token in float32; in bfloat16 every expert with its softmax weight, so that a
    # near tie between two router logits cannot send a token to another expert than the plain one
    top_k = 1 if dtype == torch.float32 else 3
    arch, cfg = load_config({"architectures": ["Toy2ForCausalLM"], "top_k": top_k})
    model = build_model(cfg, dtype, torch.device(DEV))
    assert [type(n).__name__ for n in model.cache_needs] == ["KVNeed", "KVNeed"]
    assert model.cache_needs[0].window is None and model.cache_needs[1].window == 24
    sd = random_state_dict(model.param_specs(), seed=5, dtype=torch.float32)
    assert "A.at.position.table" in sd and "A.ff.router" in sd
    sd["A.at.position.table"] = sd["A.at.position.table"] * 20      # the position term decides the scores
    sd["A.ff.router"] = sd["A.ff.router"] * 30
    if dtype == torch.bfloat16:
        sd = {k: (v.to(torch.bfloat16) if v.dim() > 1 else v) for k, v in sd.items()}
    model.build_kernels()
    model.load({k: v.to(DEV) for k, v in sd.items()})
    runner = ModelRunner(model, page_tokens=8, num_pages=16, max_requests=2)
    toks = torch.randint(0, 101, (45,), generator=torch.Generator().manual_seed(4)).tolist()
    want = plain_toy_model_2(cfg.__dict__, {n: t.float() for n, t in sd.items()}, toks)
    tol = 3e-5 if dtype == torch.float32 else 0.05
    for cuts in ([45], [13, 2, 22] + [1] * 8, [40, 5]):
        h = runner.cache.add_request()
        got, i = [], 0
        for n in cuts:
            assert runner.cache.reserve(h, n)
            got.append(runner.step([StepEntry(h, toks[i:i + n], list(range(n)))]).float().cpu())
            i += n
        runner.cache.free(h)
        err = (torch.cat(got) - want).abs().max().item()
        assert err <= tol * max(1.0, want.abs().max().item()), (dtype, cuts, err)


# ------------------------------------------------------------------ a compressed cache tensor, a capturable state, other tensor names
def make_toy_latent_mixer_class():
    from paged_batch_engine_b200.parts import CacheTensor, Mixer, PagedNeed
    from paged_batch_engine_b200.weights import ParamSpec

    class ToyLatentMixer(Mixer):
        """One compressed tensor per token in the pages instead of keys and values: c_t = x_t C^T
        (``rank`` numbers); y_t = (sum_j softmax_j(q_t . c_j) c_j) U^T over j <= t with q_t = x_t Q^T."""

        def __init__(self, hidden_size, rank, dtype, device):
            self.d, self.r, self.dtype, self.device = hidden_size, rank, dtype, device

        def cache_need(self):
            return PagedNeed((CacheTensor("latent", 1, self.r),))

        def param_specs(self, prefix):
            return [ParamSpec(prefix + "C", (self.r, self.d)), ParamSpec(prefix + "Q", (self.r, self.d)),
                    ParamSpec(prefix + "U", (self.d, self.r))]

        def load(self, tensors, prefix):
            self.C, self.Q, self.U = (tensors.pop(prefix + n).float() for n in "CQU")

        def forward(self, x, ctx, cache):
            pages = cache.tensors["latent"]                       # [page, 1, page_tokens, rank]
            P = ctx.page_tokens
            xf = x.float()
            c, q = xf @ self.C.t(), xf @ self.Q.t()
            slots = ctx.group(cache.group).slots.long()
            pages.view(-1, self.r)[slots] = c.to(pages.dtype)     # heads = 1: slot = page * P + offset
            y = torch.empty_like(xf)
            table = ctx.group(cache.group).block_table
            for r in range(ctx.num_requests):
                lo, n, before = int(ctx.q_start_host[r]), int(ctx.q_len_host[r]), int(ctx.context_before_host[r])
                total = before + n
                ids = table[r, :(total + P - 1) // P].long()
                lat = pages[ids, 0].reshape(-1, self.r)[:total].float()
                s = q[lo:lo + n] @ lat.t()
                keep = torch.arange(total, device=x.device)[None, :] <= (before + torch.arange(n, device=x.device))[:, None]
                w = torch.softmax(s.masked_fill(~keep, float("-inf")), dim=-1)
                y[lo:lo + n] = (w @ lat) @ self.U.t()
            return y.to(x.dtype)

    return ToyLatentMixer


def make_toy_device_state_mixer_class():
    from paged_batch_engine_b200.parts import Mixer, StateNeed
    from paged_batch_engine_b200.weights import ParamSpec

    class ToyDeviceStateMixer(Mixer):
        """s_t = decay * s_{t-1} + x_t * w, y_t = s_t, with the state in the request's slot.  It
        never zeroes its state (the step function does, before a request's first tokens) and it
        steps decoded tokens with device tensors only, so it says it can be captured."""
        decode_capturable = True

        def __init__(self, hidden_size, dtype, device, decay=0.5):
            self.d, self.decay = hidden_size, decay

        def cache_need(self):
            return StateNeed((self.d,), torch.float32)

        def param_specs(self, prefix):
            return [ParamSpec(prefix + "mix", (self.d,))]

        def load(self, tensors, prefix):
            self.w = tensors.pop(prefix + "mix").float()

        def forward(self, x, ctx, cache):
            if getattr(ctx, "captured", False) or int(ctx.q_len_host.max()) == 1:
                slots = ctx.state_slots[:x.shape[0]].long()       # padding rows point at the spare row
                s = cache.state[slots] * self.decay + x.float() * self.w
                cache.state.index_copy_(0, slots, s)
                return s.to(x.dtype)
            y = torch.empty_like(x)
            for r in range(ctx.num_requests):
                lo, n = int(ctx.q_start_host[r]), int(ctx.q_len_host[r])
                s = cache.state[int(ctx.state_slots_host[r])]
                for t in range(lo, lo + n):
                    s.mul_(self.decay).add_(x[t].float() * self.w)
                    y[t] = s.to(x.dtype)
            return y

    return ToyDeviceStateMixer


def plain_toy_model_3(c, w, tokens):
    T = len(tokens)
    x = plain.embedding(tokens, w["emb"]) * c["embed_scale"]
    # block A: the latent mixer, SwiGLU under other tensor names
    if c["latent"]:
        h = plain.rmsnorm(x, w["A.n1.weight"], c["eps"])
        lat, q = h @ w["A.mx.C"].t(), h @ w["A.mx.Q"].t()
        s = (q @ lat.t()).masked_fill(torch.arange(T)[None, :] > torch.arange(T)[:, None], float("-inf"))
        x = x + (torch.softmax(s, dim=-1) @ lat) @ w["A.mx.U"].t()
        f = plain.rmsnorm(x, w["A.n2.weight"], c["eps"])
        x = x + plain.linear(plain.swiglu(plain.linear(f, w["A.ff.w1.weight"]), plain.linear(f, w["A.ff.w3.weight"])),
                             w["A.ff.w2.weight"])
    # block B: the state mixer
    h = plain.rmsnorm(x, w["B.n1.weight"], c["eps"])
    st, out = torch.zeros(c["d"]), []
    for t in range(T):
        st = c["decay"] * st + h[t] * w["B.mx.mix"]
        out.append(st.clone())
    x = x + torch.stack(out)
    f = plain.rmsnorm(x, w["B.n2.weight"], c["eps"])
    x = x + plain.linear(plain.swiglu(plain.linear(f, w["B.ff.w1.weight"]), plain.linear(f, w["B.ff.w3.weight"])),
                         w["B.ff.w2.weight"])
    # block C: attention under other tensor names
    h = plain.rmsnorm(x, w["C.n1.weight"], c["eps"])
    ww = {"q_proj": "wq", "k_proj": "wk", "v_proj": "wv", "o_proj": "wo"}
    renamed = {f"C.at.{old}.{kind}": w[f"C.at.{new}.{kind}"] for old, new in ww.items() for kind in ("weight", "bias")
               if f"C.at.{new}.{kind}" in w}
    acfg = dict(num_attention_heads=c["heads"], num_key_value_heads=c["kv"], head_dim=c["hd"], hidden_size=c["d"],
                rope_theta=c["theta"])
    x = x + plain.attention_block(h, torch.arange(T), renamed, "C.at.", acfg, None)
    f = plain.rmsnorm(x, w["C.n2.weight"], c["eps"])
    x = x + plain.linear(plain.swiglu(plain.linear(f, w["C.ff.w1.weight"]), plain.linear(f, w["C.ff.w3.weight"])),
                         w["C.ff.w2.weight"])
    logits = plain.linear(plain.rmsnorm(x, w["fn.weight"], c["eps"]), w["head"])
    return c["cap"] * torch.tanh(logits / c["cap"])


@pytest.mark.parametrize("latent", [True, False], ids=["latent", "capturable"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_toy_compressed_cache_capturable_state_other_names_and_a_builder(dtype, latent):
    """Defined here, with no change to the package: a mixer whose pages hold ONE compressed
    tensor (no keys, no values; it runs host logic, so its model's decode steps stay eager); a
    mixer with state that never zeroes it (the step function does) and that, with attention
    alone beside it, keeps captured decode steps on for its model; attention and feed-forward
    reading checkpoints with other tensor names; and an architecture with a builder of its own
    (embedding scale and a cap on the logits around the generic decoder)."""
    from paged_batch_engine_b200.config import (BlockSpec, ModelSpec, PartSpec, RunStep, load_config,
                                                register_architecture)
    from paged_batch_engine_b200.engine.batch import StepEntry
    from paged_batch_engine_b200.engine.runner import ModelRunner, build_model
    from paged_batch_engine_b200.models.decoder import DecoderModel
    from paged_batch_engine_b200.parts import register_part
    from paged_batch_engine_b200.weights import random_state_dict

    register_part("mixer", "toy_latent", make_toy_latent_mixer_class(), replace=True)
    register_part("mixer", "toy_device_state", make_toy_device_state_mixer_class(), replace=True)

    @dataclass
    class Toy3Config:
        d: int = 40
        rank: int = 12
        heads: int = 4
        kv: int = 2
        hd: int = 16
        inter: int = 56
        vocab: int = 89
        eps: float = 1e-5
        theta: float = 700.0
        decay: float = 0.6
        embed_scale: float = 3.0
        cap: float = 4.0
        latent: bool = True

        @classmethod
        def from_dict(cls, d):
            return cls(**{k: v for k, v in d.items() if k in cls.__dataclass_fields__})

        def model_spec(self):
            norm = PartSpec("rmsnorm", dict(size=self.d, eps=self.eps))
            ffn = PartSpec("swiglu", dict(hidden_size=self.d, intermediate_size=self.inter,
                                          tensor_names=dict(gate="w1", down="w2", up="w3")))
            attn = PartSpec("attention", dict(hidden_size=self.d, num_heads=self.heads, num_kv_heads=self.kv,
                                              head_dim=self.hd, tensor_names=dict(q="wq", k="wk", v="wv", o="wo"),
                                              position=PartSpec("rope", dict(theta=self.theta, head_dim=self.hd))))
            names = dict(norm_mixer="n1.", norm_feed_forward="n2.", feed_forward="ff.", mixer="mx.")
            blocks = (BlockSpec("prenorm", PartSpec("toy_latent", dict(hidden_size=self.d, rank=self.rank)), ffn, norm,
                                norm, "A.", names),
                      BlockSpec("prenorm", PartSpec("toy_device_state", dict(hidden_size=self.d, decay=self.decay)), ffn,
                                norm, norm, "B.", names),
                      BlockSpec("prenorm", attn, ffn, norm, norm, "C.", dict(names, mixer="at.")))
            if not self.latent:
                blocks = blocks[1:]
            run = tuple(RunStep(i, i) for i in range(len(blocks)))
            return ModelSpec("Toy3ForCausalLM", self.d, self.vocab, blocks, run, norm, "emb", "fn.", "head", 512)

    conf = Toy3Config(latent=latent)

    class ScaledCappedDecoder(DecoderModel):
        """The generic decoder with the embedding table scaled at load and the logits capped."""

        def load(self, tensors):
            super().load(tensors)
            self.embed = (self.embed.float() * conf.embed_scale).to(self.embed.dtype)

        def forward(self, ctx, storage):
            logits = super().forward(ctx, storage)
            return conf.cap * torch.tanh(logits / conf.cap)

    register_architecture("Toy3ForCausalLM", Toy3Config, builder=lambda spec, dt, dev: ScaledCappedDecoder(spec, dt, dev),
                          replace=True)
    model = build_model({"architectures": ["Toy3ForCausalLM"], "latent": latent}, dtype, torch.device(DEV))
    assert type(model).__name__ == "ScaledCappedDecoder"
    assert [type(n).__name__ for n in model.cache_needs] == (["PagedNeed"] if latent else []) + ["StateNeed", "KVNeed"]
    names = [p.name for p in model.param_specs()]
    assert "C.at.wq.weight" in names and "B.ff.w3.weight" in names and not any("q_proj" in n or "gate_proj" in n for n in names)
    sd = random_state_dict(model.param_specs(), seed=9, dtype=torch.float32)
    for k in sd:
        if k.endswith(("mx.C", "mx.Q", "wq.weight", "wk.weight")):
            sd[k] = sd[k] * 12
        if k.endswith("mix"):
            sd[k] = torch.linspace(0.5, 1.5, conf.d)
    sd["head"] = sd["head"] * 8                                     # logits large enough for the cap to bend them
    if dtype == torch.bfloat16:
        sd = {k: (v.to(torch.bfloat16) if v.dim() > 1 else v) for k, v in sd.items()}
    model.build_kernels()
    model.load({k: v.to(DEV) for k, v in sd.items()})
    runner = ModelRunner(model, page_tokens=8, num_pages=24, max_requests=4)
    if latent:
        assert len(runner.storage.groups) == 2                      # the latent pages and the keys/values
        assert [t.name for t in runner.storage.groups[0].tensors] == ["latent"]
        assert runner.storage.bytes_per_token() == (conf.rank + 2 * conf.kv * conf.hd) * (4 if dtype == torch.float32 else 2)
    gen = torch.Generator().manual_seed(6)
    toks = {r: torch.randint(0, conf.vocab, (n,), generator=gen).tolist() for r, n in (("a", 41), ("b", 19), ("c", 30))}
    plain_w = {n: t.float() for n, t in sd.items()}
    want = {r: plain_toy_model_3(conf.__dict__, plain_w, t) for r, t in toks.items()}
    assert max(v.abs().max().item() for v in want.values()) > 0.6 * conf.cap
    tol = 3e-5 if dtype == torch.float32 else 0.05
    # the state rows start dirty: the step function must zero them for every new request
    for t in runner.storage.state.values():
        t.fill_(7.0)
    for graphs in (False, True):
        handles = {r: runner.cache.add_request() for r in toks}
        got = {r: [] for r in toks}
        heads = {"a": 30, "b": 9, "c": 21}
        for r in toks:                                              # prompt portions, two steps each
            done = 0
            for n in (heads[r] - 4, 4):
                assert runner.cache.reserve(handles[r], n)
                got[r].append(runner.step([StepEntry(handles[r], toks[r][done:done + n], list(range(n)))]).float().cpu())
                done += n
        pos = dict(heads)
        while any(pos[r] < len(toks[r]) for r in toks):             # all live requests decode together
            live = [r for r in toks if pos[r] < len(toks[r])]
            for r in live:
                assert runner.cache.reserve(handles[r], 1)
            out = runner.step([StepEntry(handles[r], [toks[r][pos[r]]], [0]) for r in live], decode_graph=graphs).float().cpu()
            for i, r in enumerate(live):
                got[r].append(out[i:i + 1])
                pos[r] += 1
        for r in toks:
            runner.cache.free(handles[r])
            err = (torch.cat(got[r]) - want[r]).abs().max().item()
            assert err <= tol * max(1.0, want[r].abs().max().item()), (dtype, graphs, r, err)
    # the state mixer and attention can be captured; the latent mixer's host logic cannot
    assert runner.graphs.eligible([StepEntry(0, [1], [0])]) == (not latent)
    assert (runner.graphs.replays > 0) == (not latent)
    runner.cache.check_invariants()


# ------------------------------------------------------------------ position ids that are not the place in the sequence
def make_toy_grid_position_class():
    from paged_batch_engine_b200.parts import PositionEncoding
    from paged_batch_engine_b200.weights import ParamSpec

    class ToyGridPosition(PositionEncoding):
        """Two axes of position ids (a row and a column, say): q and k get the learned vector of
        each axis added.  The ids come with the step's entries, not from the place in the sequence."""
        applies_itself = True

        def __init__(self, head_dim, rows, cols, dtype, device):
            self.hd, self.rows, self.cols = head_dim, rows, cols

        def param_specs(self, prefix):
            return [ParamSpec(prefix + "row_table", (self.rows, self.hd)), ParamSpec(prefix + "col_table", (self.cols, self.hd))]

        def load(self, tensors, prefix):
            self.rt = tensors.pop(prefix + "row_table").float()
            self.ct = tensors.pop(prefix + "col_table").float()

        def apply(self, q, k, positions):
            assert positions.dim() == 2 and positions.shape[1] == 2
            add = (self.rt[positions[:, 0].long()] + self.ct[positions[:, 1].long()]).unsqueeze(1)
            return q + add, k + add

    return ToyGridPosition


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_position_ids_brought_by_the_entries(dtype):
    """Position ids that a step's entries bring: two axes for a position encoding with code of
    its own (defined here), and one axis for the rotary kernel (ids shifted against the place in
    the sequence).  The cache and the causal mask still go by the place in the sequence."""
    from paged_batch_engine_b200.config import PartSpec
    from paged_batch_engine_b200.cache.storage import CacheStorage
    from paged_batch_engine_b200.engine.batch import StepEntry
    from paged_batch_engine_b200.parts import build_part, register_part
    register_part("position", "toy_grid", make_toy_grid_position_class(), replace=True)
    torch.manual_seed(3)
    d, H, KV, hd, T, P = 64, 4, 2, 32, 37, 8
    cfg = dict(num_attention_heads=H, num_key_value_heads=KV, head_dim=hd, hidden_size=d, rope_theta=900.0)
    tol = 3e-5 if dtype == torch.float32 else 0.04
    x = torch.randn(T, d).to(dtype)
    for kind in ("grid", "shifted"):
        position = PartSpec("toy_grid", dict(head_dim=hd, rows=8, cols=5)) if kind == "grid" else \
            PartSpec("rope", dict(theta=900.0, head_dim=hd))
        att = build_part("mixer", PartSpec("attention", dict(hidden_size=d, num_heads=H, num_kv_heads=KV, head_dim=hd,
                                                             position=position)), dtype, DEV)
        w = {p.name: (torch.randn(p.shape) * (0.3 if len(p.shape) > 1 else 0.1)).to(dtype if len(p.shape) > 1 else torch.float32)
             for p in att.param_specs("a.")}
        att.load({k: v.to(DEV) for k, v in w.items()}, "a.")
        wf = {k: v.float() for k, v in w.items()}
        if kind == "grid":
            ids = torch.stack([torch.arange(T) // 5, torch.arange(T) % 5], dim=1)
            q = plain.linear(x.float(), wf["a.q_proj.weight"], wf["a.q_proj.bias"]).view(T, H, hd)
            k = plain.linear(x.float(), wf["a.k_proj.weight"], wf["a.k_proj.bias"]).view(T, KV, hd)
            v = plain.linear(x.float(), wf["a.v_proj.weight"], wf["a.v_proj.bias"]).view(T, KV, hd)
            add = (wf["a.position.row_table"][ids[:, 0]] + wf["a.position.col_table"][ids[:, 1]]).unsqueeze(1)
            o = plain.causal_attention(q + add, k + add, v, hd ** -0.5)
            want = plain.linear(o.reshape(T, H * hd), wf["a.o_proj.weight"])
        else:
            ids = torch.arange(T) + 100 + (torch.arange(T) // 9) * 3          # neither the place nor a plain shift
            want = plain.attention_block(x.float(), ids, wf, "a.", cfg, None)
        storage = CacheStorage([att.cache_need()], P, 8, 2, dtype, torch.device(DEV), poison=True)
        keys = [(0,) + kk for kk in att.work_keys()]
        for cuts in ([T], [11, 2, 19] + [1] * 5):
            hnd = storage.manager.add_request()
            outs, i = [], 0
            for n in cuts:
                assert storage.manager.reserve(hnd, n)
                ctx = _ctx(storage.manager, [StepEntry(hnd, [0] * n, position_ids=ids[i:i + n].tolist())], keys)
                assert ctx.position_ids.shape == ((n, 2) if kind == "grid" else (n,))
                assert ctx.positions.tolist() == list(range(i, i + n))
                outs.append(att.forward(x[i:i + n].to(DEV), ctx, storage.layer(0)).float().cpu())
                storage.manager.commit(hnd, n)
                i += n
            storage.manager.free(hnd)
            got = torch.cat(outs)
            assert (got - want).abs().max() <= tol * max(1.0, want.abs().max()), (kind, cuts)
