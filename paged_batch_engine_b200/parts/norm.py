"""RMSNorm fused with the residual add that precedes it."""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights.loader import ParamSpec
from .base import Norm, register_part


class RMSNorm(Norm):
    """y = (w * x) * rsqrt(mean(x^2) + eps) on x = residual + delta, all in float32.

    The reference runs the add (add_kernel.cu:6-15) and the norm (rmsnorm_kernel.cu:9-41)
    as two launches and rounds the residual stream to the run dtype in between; here it is
    one launch and the residual stream stays float32."""

    def __init__(self, size: int, eps: float, dtype, device, weight_name: str = "weight"):
        self.size, self.eps, self.dtype, self.device = int(size), float(eps), dtype, device
        self.weight_name = weight_name
        self.gain = None

    def param_specs(self, prefix):
        return [ParamSpec(prefix + self.weight_name, (self.size,))]

    def load(self, tensors, prefix):
        self.gain = tensors[prefix + self.weight_name].to(torch.float32).contiguous()

    def add_norm(self, residual, delta, rows=None, out_dtype=None):
        n = residual.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.size), dtype=out_dtype or self.dtype, device=residual.device)
        return ops.add_rmsnorm(residual, delta, self.gain, out, self.eps, rows)


register_part("norm", "rmsnorm", RMSNorm, replace=True)
