"""Grouped-query attention over the paged cache."""
from __future__ import annotations

from typing import Optional

import torch

from ..config.specs import PartSpec
from ..csrc import ops

from ..weights.loader import ParamSpec
from .base import KVNeed, Mixer, build_part, register_part


class GQAttention(Mixer):
    """q, k, v = x W^T (+ b) as one fused product; position encoding on q and k; k and v
    written to the cache; causal attention of every row over its request's pages (all
    keys, or the last ``window``); output projection.

    Reference: infMain/source/model/qwen2_batch.cpp:604-750 (three products, three bias
    launches, rope, scatter, decode and prefill attention kernels, output product).
    Checkpoint tensors: {q,k,v}_proj.weight [heads*head_dim, hidden] (+ .bias),
    o_proj.weight [hidden, heads*head_dim] (+ .bias when o_bias).  ``tensor_names`` renames
    the four projections for checkpoints that call them otherwise, e.g.
    ``dict(q="wq", k="wk", v="wv", o="wo")``; ``.weight`` / ``.bias`` are appended."""
    TENSOR_NAMES = dict(q="q_proj", k="k_proj", v="v_proj", o="o_proj")
    decode_capturable = True      # decoded tokens are stepped from the step's device arrays alone

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 dtype, device, qkv_bias: bool = True, o_bias: bool = False,
                 scale: Optional[float] = None, window: Optional[int] = None,
                 position: Optional[PartSpec] = None, kernel: Optional[str] = None,
                 tensor_names: Optional[dict] = None):
        unknown = set(tensor_names or {}) - set(self.TENSOR_NAMES)
        if unknown:
            raise ValueError(f"tensor_names knows q, k, v and o; got {sorted(unknown)}")
        self.names = dict(self.TENSOR_NAMES, **(tensor_names or {}))
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.head_dim, self.qkv_bias, self.o_bias = head_dim, qkv_bias, o_bias
        self.scale = float(scale) if scale is not None else head_dim ** -0.5
        self.window = int(window) if window else None
        self.dtype, self.device = dtype, device
        self.position = build_part("position", position, dtype, device) if position is not None \
            else build_part("position", PartSpec("none"), dtype, device)
        self.kernel_kind, self.tile_rows, self.key_tile = ops.attention_kernel_config(head_dim, dtype, kernel)
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = None

    # ---- what it keeps
    def cache_need(self):
        return KVNeed(self.num_kv_heads, self.head_dim, self.window)

    def work_keys(self):
        return [(self.num_heads // self.num_kv_heads, self.tile_rows, self.window)]

    def kernel_libraries(self, dtype):
        return [("elementwise", None), ("rope_kv", None)] + ops.gemm_libraries(dtype) + \
            ops.attention_libraries(self.head_dim, dtype)

    # ---- tensors
    def param_specs(self, prefix):
        q_out, kv_out = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        n = self.names
        specs = [ParamSpec(prefix + n["q"] + ".weight", (q_out, self.hidden_size)),
                 ParamSpec(prefix + n["k"] + ".weight", (kv_out, self.hidden_size)),
                 ParamSpec(prefix + n["v"] + ".weight", (kv_out, self.hidden_size)),
                 ParamSpec(prefix + n["o"] + ".weight", (self.hidden_size, q_out))]
        if self.qkv_bias:
            specs += [ParamSpec(prefix + n["q"] + ".bias", (q_out,)),
                      ParamSpec(prefix + n["k"] + ".bias", (kv_out,)),
                      ParamSpec(prefix + n["v"] + ".bias", (kv_out,))]
        if self.o_bias:
            specs.append(ParamSpec(prefix + n["o"] + ".bias", (self.hidden_size,)))
        return specs + self.position.param_specs(prefix + "position.")

    def load(self, tensors, prefix):
        nm = self.names
        ws = [tensors.pop(prefix + nm[n] + ".weight") for n in "qkv"]
        if len({w.dtype for w in ws}) != 1:
            ws = [w.to(torch.float32) for w in ws]
        self.w_qkv = torch.cat(ws, dim=0).contiguous()
        del ws
        if self.qkv_bias:
            self.b_qkv = torch.cat([tensors.pop(prefix + nm[n] + ".bias").to(torch.float32)
                                    for n in "qkv"]).contiguous()
        self.w_o = tensors.pop(prefix + nm["o"] + ".weight").contiguous()
        if self.o_bias:
            self.b_o = tensors.pop(prefix + nm["o"] + ".bias").to(torch.float32).contiguous()
        self.position.load(tensors, prefix + "position.")

    # ---- compute
    def fused_decode_splits(self, meta, cache, inv_freq, rotary_dim, interleaved) -> int:
        """Blocks per (request, key/value head) for the fused decode kernel, 0: not this step."""
        H, KV, hd = self.num_heads, self.num_kv_heads, self.head_dim
        if not (meta.decode_rows > 0 and cache.writes and inv_freq is not None and rotary_dim == hd
                and not interleaved and self.kernel_kind != "simple"
                and ops.fused_decode_attention_applies(self.dtype, hd, H // KV)):
            return 0
        return ops.fused_decode_splits(meta.decode_rows, KV, meta.longest_keys, meta.q_len.device)

    def _apply_position(self, qkv, positions):
        T = qkv.shape[0]
        H, KV, hd = self.num_heads, self.num_kv_heads, self.head_dim
        f = qkv.float()
        if self.b_qkv is not None:
            f = f + self.b_qkv
        q, k = self.position.apply(f[:, :H * hd].reshape(T, H, hd), f[:, H * hd:(H + KV) * hd].reshape(T, KV, hd),
                                   positions)
        return torch.cat([q.reshape(T, H * hd), k.reshape(T, KV * hd), f[:, (H + KV) * hd:]], dim=1).to(self.dtype)

    def forward(self, x, ctx, cache):
        T = x.shape[0]
        H, KV, hd = self.num_heads, self.num_kv_heads, self.head_dim
        qkv = ops.linear(x, self.w_qkv, None, out_dtype=self.dtype, kind=1)
        bias = self.b_qkv
        if self.position.applies_itself:
            # a position encoding with code of its own: it gets q and k with the bias added and
            # the kernel below only copies (no rotation, no bias)
            qkv, bias = self._apply_position(qkv, ctx.position_ids), None
            inv_freq, rotary_dim, interleaved = None, 0, False
            kernel_positions = ctx.positions          # the kernels below only copy
        else:
            inv_freq, rotary_dim, interleaved = self.position.kernel_args()
            kernel_positions = ctx.position_ids
        if ctx.position_ids.dim() != 1 and not self.position.applies_itself:
            raise ValueError("position ids with several axes need a position encoding with code of its own")
        group = ctx.group(cache.group)
        k_pages, v_pages = cache.k, cache.v
        meta = ctx.attention_work(cache.group, H // KV, self.tile_rows, self.window, H, hd)
        splits = self.fused_decode_splits(meta, cache, inv_freq, rotary_dim, interleaved)
        if splits:
            # decoded tokens only, every block of the step resident at once: position encoding, cache
            # write, attention and the merge of the key splits in one launch
            out = torch.empty((T, H * hd), dtype=self.dtype, device=x.device)
            ops.attention_decode_fused(qkv, bias, k_pages, v_pages, out, meta, kernel_positions, group.slots,
                                       inv_freq, meta.decode_rows, H, KV, hd, self.scale, self.window,
                                       ctx.page_tokens, splits=splits)
            return ops.linear(out, self.w_o, self.b_o, out_dtype=self.dtype, kind=2)
        q = torch.empty((T, H * hd), dtype=self.dtype, device=x.device)
        ops.rope_kv_write(qkv, bias, q, k_pages if cache.writes else None,
                          v_pages if cache.writes else None, kernel_positions, group.slots, inv_freq,
                          H, KV, hd, rotary_dim, ctx.page_tokens, interleaved)
        out = torch.empty((T, H * hd), dtype=self.dtype, device=x.device)
        ops.paged_attention(q, k_pages, v_pages, out, meta, H, KV, hd, self.scale, self.window,
                            ctx.page_tokens, kind=self.kernel_kind)
        return ops.linear(out, self.w_o, self.b_o, out_dtype=self.dtype, kind=2)


register_part("mixer", "attention", GQAttention, replace=True)
