"""Dense gated feed-forward."""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights.loader import ParamSpec
from .base import FeedForward, register_part


class SwiGLU(FeedForward):
    """m = (silu(x W_gate^T) * (x W_up^T)) W_down^T, no biases; gate and up are one fused
    product.  Reference: infMain/source/model/qwen2_batch.cpp:762-777 and
    swiglu_kernel.cu:6-25 (g * 1/(1+exp(-g)) * u in float32).
    Checkpoint tensors: gate_proj.weight, up_proj.weight [inter, hidden]; down_proj.weight
    [hidden, inter]; ``tensor_names`` renames them, e.g. ``dict(gate="w1", down="w2", up="w3")``."""
    TENSOR_NAMES = dict(gate="gate_proj", up="up_proj", down="down_proj")

    def __init__(self, hidden_size: int, intermediate_size: int, dtype, device, tensor_names=None):
        unknown = set(tensor_names or {}) - set(self.TENSOR_NAMES)
        if unknown:
            raise ValueError(f"tensor_names knows gate, up and down; got {sorted(unknown)}")
        self.names = dict(self.TENSOR_NAMES, **(tensor_names or {}))
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.dtype, self.device = dtype, device
        self.w_gate_up = self.w_down = None

    def kernel_libraries(self, dtype):
        return [("elementwise", None)] + ops.gemm_libraries(dtype, 2 * self.intermediate_size * self.hidden_size)

    def param_specs(self, prefix):
        i, h = self.intermediate_size, self.hidden_size
        n = self.names
        return [ParamSpec(prefix + n["gate"] + ".weight", (i, h)),
                ParamSpec(prefix + n["up"] + ".weight", (i, h)),
                ParamSpec(prefix + n["down"] + ".weight", (h, i))]

    def load(self, tensors, prefix):
        n = self.names
        g, u = tensors.pop(prefix + n["gate"] + ".weight"), tensors.pop(prefix + n["up"] + ".weight")
        if g.dtype != u.dtype:
            g, u = g.to(torch.float32), u.to(torch.float32)
        self.w_gate_up = torch.cat([g, u], dim=0).contiguous()
        del g, u
        self.w_down = tensors.pop(prefix + n["down"] + ".weight").contiguous()

    def forward(self, x, ctx):
        # few rows (decode): the activation is the epilogue of a weight-streaming product
        if ops.stream_applies(x, self.w_gate_up, 4):
            act = ops.gemm_stream(x, self.w_gate_up, self.dtype, swiglu=True)
            return ops.linear(act, self.w_down, None, out_dtype=self.dtype, kind=8)
        if ops.skinny_applies(x, self.w_gate_up):
            act = ops.gemm_skinny(x, self.w_gate_up, None, self.dtype, swiglu=True)
            return ops.linear(act, self.w_down, None, out_dtype=self.dtype, kind=8)
        if ops.tc5_applies(x, self.w_gate_up, 4):
            act = ops.gemm_tc5(x, self.w_gate_up, self.dtype, swiglu=True)
            return ops.linear(act, self.w_down, None, out_dtype=self.dtype, kind=8)
        gu = ops.linear(x, self.w_gate_up, None, out_dtype=self.dtype, kind=32)
        act = torch.empty((x.shape[0], self.intermediate_size), dtype=self.dtype, device=x.device)
        ops.silu_mul(gu, act)
        return ops.linear(act, self.w_down, None, out_dtype=self.dtype, kind=8)


register_part("feed_forward", "swiglu", SwiGLU, replace=True)
