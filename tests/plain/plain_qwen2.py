"""Plain, slow implementation of the Qwen2.5 dense decoder: the tests' oracle.

Whole sequences, no cache, no paging, one function for each part, float32 (or
float64 when asked) on the CPU with elementary torch tensor arithmetic.  It
shares no code with the engine: it reads ``config.json`` as a plain dict and
weights as a plain ``{name: tensor}`` dict with the checkpoint's own tensor
names.

Every function is written from the formulas of the reference engine
(Destination2020/Paged-Batch-Engine); each docstring cites the file and lines
of the reference that the formula was taken from.  The structure (pre-norm
placement, q/k/v bias, GQA, SwiGLU, tied head) is additionally anchored once
against the reference's own ``tools/model_qwen2.py`` on a tiny random model
(``tests/golden/make_reference_golden.py``); rotation pairing, theta, eps, the
untied head and the sliding window rest on the formulas alone, because the
reference's Python model differs from its C++ engine in those.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch

Tensor = torch.Tensor


def embedding(token_ids: Sequence[int], table: Tensor) -> Tensor:
    """x[t, :] = E[id[t], :], a pure row copy without scaling.

    Reference: infMain/source/op/kernels/cuda/emb_kernel.cu:5-23.
    """
    idx = torch.as_tensor(list(token_ids), dtype=torch.long)
    return table[idx].clone()


def rmsnorm(x: Tensor, gain: Tensor, eps: float) -> Tensor:
    """y_i = (w_i * x_i) * rsqrt(mean_j(x_j^2) + eps).

    Reference: infMain/source/op/kernels/cuda/rmsnorm_kernel.cu:9-41 (sum of
    squares, division by the row size, ``rsqrtf(mean + eps)``, then the triple
    product ``w * x * scale`` evaluated left to right).
    """
    mean_sq = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    scale = torch.rsqrt(mean_sq + eps)
    return (gain * x) * scale


def rope_inv_freq(head_dim: int, theta: float, dtype=torch.float32) -> Tensor:
    """freq_i = 1 / theta^(2i / head_dim) for pair index i in [0, head_dim/2).

    Reference: infMain/source/op/kernels/cuda/rope_kernel.cu:69-94 builds the
    table entry ``d`` as ``1/powf(theta, d/head_size)`` and the batched kernel
    reads entry ``2*i`` for pair ``i`` (rope_kernel.cu:172-176).
    """
    i = torch.arange(0, head_dim // 2, dtype=dtype)
    return 1.0 / torch.pow(torch.tensor(theta, dtype=dtype), (2.0 * i) / head_dim)


def rope_rotate_half(x: Tensor, positions: Tensor, theta: float) -> Tensor:
    """Rotate-half ("neox") pairing: (a, b) = (v[i], v[i + hd/2]);
    v[i] = a cos - b sin; v[i + hd/2] = b cos + a sin; angle = pos * freq_i.

    ``x`` is [T, heads, head_dim].  Reference:
    infMain/source/op/kernels/cuda/rope_kernel.cu:149-215 (Qwen2 branch, pair
    ``head_dim`` and ``head_dim + head_size/2``; ``fcr*v0 - fci*v1`` and
    ``fcr*v1 + fci*v0``).
    """
    hd = x.shape[-1]
    half = hd // 2
    inv_freq = rope_inv_freq(hd, theta, dtype=x.dtype)
    angle = positions.to(x.dtype)[:, None] * inv_freq[None, :]  # [T, half]
    cos = torch.cos(angle)[:, None, :]
    sin = torch.sin(angle)[:, None, :]
    a = x[..., :half]
    b = x[..., half:]
    return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)


def rope_interleaved(x: Tensor, positions: Tensor, theta: float) -> Tensor:
    """Interleaved pairing (2i, 2i+1), as the reference's Python model does.

    Only used to anchor the structure against tools/model_qwen2.py:58-80; the
    C++ engine itself uses ``rope_rotate_half``.
    """
    hd = x.shape[-1]
    inv_freq = rope_inv_freq(hd, theta, dtype=x.dtype)
    angle = positions.to(x.dtype)[:, None] * inv_freq[None, :]
    cos = torch.cos(angle)[:, None, :]
    sin = torch.sin(angle)[:, None, :]
    xr = x[..., 0::2]
    xi = x[..., 1::2]
    out_r = xr * cos - xi * sin
    out_i = xr * sin + xi * cos
    return torch.stack([out_r, out_i], dim=-1).flatten(-2)


def linear(x: Tensor, weight: Tensor, bias: Optional[Tensor] = None) -> Tensor:
    """y = x W^T (+ b), W stored [out, in] row-major.

    Reference: infMain/source/op/kernels/cuda/matmul_kernel_batch.cu:241-261
    (``Y[M,N] = X[M,K] * W[N,K]^T``) and add_bias_kernel.cu:7-18.
    """
    y = x @ weight.t()
    if bias is not None:
        y = y + bias
    return y


def causal_attention(q: Tensor, k: Tensor, v: Tensor, scale: float,
                     window: Optional[int] = None) -> Tensor:
    """Causal grouped-query attention over a whole sequence.

    q [T, H, hd]; k, v [T, KV, hd]; query head h reads kv head h // (H/KV).
    s_j = (q . k_j) * scale for keys j <= p (p the query's position); softmax
    over those keys; o = sum_j softmax_j v_j.  The causal mask is "keys above
    p are not visited".

    Reference: infMain/source/op/kernels/cuda/paged_mha_kernel.cu:363-550 (kv
    head = head / kv_mul, scale 1/sqrt(head_size), online softmax over keys
    0..seq_len-1) and paged_mha_prefill_kernel.cu:368-520.

    ``window`` (not in the reference, which always attends to every key): when
    given, a query at position p sees only keys j with p - window < j <= p.
    """
    T, H, hd = q.shape
    KV = k.shape[1]
    group = H // KV
    out = torch.empty_like(q)
    pos = torch.arange(T)
    visible = pos[None, :] <= pos[:, None]
    if window is not None:
        visible = visible & (pos[None, :] > pos[:, None] - window)
    for h in range(H):
        g = h // group
        s = (q[:, h, :] @ k[:, g, :].t()) * scale
        s = s.masked_fill(~visible, float("-inf"))
        m = s.max(dim=-1, keepdim=True).values
        e = torch.exp(s - m)
        p = e / e.sum(dim=-1, keepdim=True)
        out[:, h, :] = p @ v[:, g, :]
    return out


def swiglu(gate: Tensor, up: Tensor) -> Tensor:
    """a = (g * 1/(1+exp(-g))) * u.

    Reference: infMain/source/op/kernels/cuda/swiglu_kernel.cu:6-25.
    """
    return (gate * (1.0 / (1.0 + torch.exp(-gate)))) * up


def attention_block(h: Tensor, positions: Tensor, w: Dict[str, Tensor], prefix: str,
                    cfg: dict, window: Optional[int], rope=rope_rotate_half) -> Tensor:
    """q,k,v = h W^T + b; rope(q), rope(k); causal GQA; o W_o^T (no bias).

    Reference: infMain/source/model/qwen2_batch.cpp:604-642 (three projections,
    three bias adds, rope on q and k), :663-745 (attention), :748-750 (output
    projection without bias).
    """
    H = cfg["num_attention_heads"]
    KV = cfg["num_key_value_heads"]
    hd = cfg.get("head_dim") or cfg["hidden_size"] // H
    T = h.shape[0]
    q = linear(h, w[prefix + "q_proj.weight"], w[prefix + "q_proj.bias"]).view(T, H, hd)
    k = linear(h, w[prefix + "k_proj.weight"], w[prefix + "k_proj.bias"]).view(T, KV, hd)
    v = linear(h, w[prefix + "v_proj.weight"], w[prefix + "v_proj.bias"]).view(T, KV, hd)
    theta = float(cfg.get("rope_theta", 1000000.0))
    q = rope(q, positions, theta)
    k = rope(k, positions, theta)
    o = causal_attention(q, k, v, 1.0 / math.sqrt(hd), window)
    return linear(o.reshape(T, H * hd), w[prefix + "o_proj.weight"])


def feed_forward(f: Tensor, w: Dict[str, Tensor], prefix: str) -> Tensor:
    """m = (silu(f W1^T) * (f W3^T)) W2^T, no biases.

    Reference: infMain/source/model/qwen2_batch.cpp:762-777.
    """
    g = linear(f, w[prefix + "gate_proj.weight"])
    u = linear(f, w[prefix + "up_proj.weight"])
    return linear(swiglu(g, u), w[prefix + "down_proj.weight"])


def layer_window(cfg: dict, layer: int) -> Optional[int]:
    """The window of a layer from config.json's own keys: layers with index >=
    ``max_window_layers`` use ``sliding_window`` keys when ``use_sliding_window``
    is set.  The reference engine has no window (it always reads every key); this
    reading of the three keys is this project's."""
    if not cfg.get("use_sliding_window", False):
        return None
    if cfg.get("sliding_window") is None:
        return None
    if layer >= int(cfg.get("max_window_layers", cfg["num_hidden_layers"])):
        return int(cfg["sliding_window"])
    return None


def forward_logits(cfg: dict, w: Dict[str, Tensor], token_ids: Sequence[int],
                   dtype=torch.float32, rope=rope_rotate_half) -> Tensor:
    """Logits [T, vocab] of one whole sequence.

    Pre-norm placement: x -> norm -> attention -> +x; -> norm -> mlp -> +x;
    final norm; LM head (the embedding table when tied).  Reference:
    infMain/source/model/qwen2_batch.cpp:584-798.
    """
    w = {k: t.to(dtype) for k, t in w.items()}
    eps = float(cfg.get("rms_norm_eps", 1e-6))
    x = embedding(token_ids, w["model.embed_tokens.weight"])
    positions = torch.arange(len(token_ids))
    for layer in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{layer}."
        h = rmsnorm(x, w[p + "input_layernorm.weight"], eps)
        x = x + attention_block(h, positions, w, p + "self_attn.", cfg,
                                layer_window(cfg, layer), rope)
        f = rmsnorm(x, w[p + "post_attention_layernorm.weight"], eps)
        x = x + feed_forward(f, w, p + "mlp.")
    x = rmsnorm(x, w["model.norm.weight"], eps)
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) \
        else w["lm_head.weight"]
    return linear(x, head)


# --------------------------------------------------------------------------------------
# Sampling oracle
# --------------------------------------------------------------------------------------

def request_sample_uniform(seed: int, counter: int) -> float:
    """Counter-based SplitMix64 uniform in [0, 1) with 24 bits.

    Reference: infMain/include/serving/generation_config.h:14-20.
    """
    mask = (1 << 64) - 1
    z = (seed + 0x9E3779B97F4A7C15 * (counter + 1)) & mask
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
    z ^= z >> 31
    return float(z >> 40) * (1.0 / 16777216.0)


def sample_row(logits: Sequence[float], temperature: float = 0.0, top_k: int = 0,
               top_p: float = 1.0, repetition_penalty: float = 1.0,
               seen_tokens: Sequence[int] = (), uniform: float = 0.0) -> int:
    """The reference's host sampler, step by step.

    Greedy (temperature <= 0, top_k <= 0, top_p >= 1, penalty == 1): argmax with
    the lowest index winning ties.  Otherwise: repetition penalty on seen tokens
    (logit / p when positive, logit * p otherwise); the top_k candidates by
    (logit descending, token ascending); probabilities
    exp((logit - max) / max(T, 1e-6)) normalised in double; sort by (probability
    descending, token ascending); nucleus cut keeping candidates until the
    cumulative probability reaches top_p (at least one); inverse CDF with
    ``uniform * sum(kept)``.

    Reference: infMain/source/model/qwen2.cpp:104-203.
    """
    n = len(logits)
    vals = torch.as_tensor(logits, dtype=torch.float32).tolist()   # float32 values, as the row holds
    greedy = temperature <= 0.0 and top_k <= 0 and top_p >= 1.0 and repetition_penalty == 1.0
    if greedy:
        best, best_val = 0, vals[0]
        for i in range(1, n):
            if vals[i] > best_val:
                best, best_val = i, vals[i]
        return best
    if repetition_penalty != 1.0:
        seen = set(int(t) for t in seen_tokens)
        for i in seen:
            if 0 <= i < n:
                x = vals[i]
                x = x / repetition_penalty if x > 0.0 else x * repetition_penalty
                vals[i] = torch.tensor(x, dtype=torch.float32).item()
    cands = sorted(range(n), key=lambda i: (-vals[i], i))
    k = min(top_k, n) if top_k > 0 else n
    cands = cands[:k]
    t = max(1e-6, float(temperature))
    mx = vals[cands[0]]
    diffs = (torch.tensor([vals[i] for i in cands], dtype=torch.float32)
             - torch.tensor(mx, dtype=torch.float32)).tolist()       # float32 subtraction
    probs = {i: math.exp(d / t) for i, d in zip(cands, diffs)}
    denom = sum(probs[i] for i in cands)
    if not (denom > 0.0) or not math.isfinite(denom):
        return cands[0]
    for i in cands:
        probs[i] /= denom
    cands = sorted(cands, key=lambda i: (-probs[i], i))
    if top_p < 1.0:
        cum = 0.0
        keep = 0
        while keep < len(cands):
            cum += probs[cands[keep]]
            keep += 1
            if cum >= top_p:
                break
        cands = cands[:max(1, keep)]
    weight_sum = sum(probs[i] for i in cands)
    draw = float(uniform) * weight_sum
    for i in cands:
        draw -= probs[i]
        if draw <= 0.0:
            return i
    return cands[-1]


def sample_cdf_interval(logits: Sequence[float], token: int, temperature: float, top_k: int = 0,
                        top_p: float = 1.0):
    """[lo, hi) of ``token`` on the reference's inverse-CDF axis (in units of the kept
    mass), or None if the token is not among the kept candidates.  Lets a test state
    how far a uniform draw lies from a decision boundary."""
    n = len(logits)
    vals = torch.as_tensor(logits, dtype=torch.float32).tolist()
    cands = sorted(range(n), key=lambda i: (-vals[i], i))
    k = min(top_k, n) if top_k > 0 else n
    cands = cands[:k]
    t = max(1e-6, float(temperature))
    mx = vals[cands[0]]
    probs = {i: math.exp((vals[i] - mx) / t) for i in cands}
    denom = sum(probs.values())
    for i in cands:
        probs[i] /= denom
    cands = sorted(cands, key=lambda i: (-probs[i], i))
    if top_p < 1.0:
        cum, keep = 0.0, 0
        while keep < len(cands):
            cum += probs[cands[keep]]
            keep += 1
            if cum >= top_p:
                break
        cands = cands[:max(1, keep)]
    total = sum(probs[i] for i in cands)
    lo = 0.0
    for i in cands:
        hi = lo + probs[i] / total
        if i == token:
            return lo, hi
        lo = hi
    return None


def greedy_generate(cfg: dict, w: Dict[str, Tensor], prompt: Sequence[int], max_new_tokens: int,
                    eos_ids: Sequence[int] = (), dtype=torch.float32) -> List[int]:
    """Greedy generation by recomputing the whole sequence for every token.

    Stops on EOS (not appended) or after ``max_new_tokens`` sampled tokens, as the
    reference's scheduler does (infMain/source/serving/scheduler.cpp:84-107).
    """
    seq = list(prompt)
    out: List[int] = []
    for _ in range(max_new_tokens):
        logits = forward_logits(cfg, w, seq, dtype=dtype)[-1]
        tok = int(torch.argmax(logits))  # torch.argmax returns the first maximal index
        if tok in eos_ids:
            break
        out.append(tok)
        seq.append(tok)
    return out
