"""Rotary position encoding as data for the kernel that applies it."""
from __future__ import annotations

import torch

from .base import PositionEncoding, register_part


class RotaryEncoding(PositionEncoding):
    """angle(pos, i) = pos * theta^(-2i / rotary_dim) for pair i; pairs are
    (i, i + rotary_dim/2) ("half", the reference's Qwen2 branch,
    rope_kernel.cu:163-176) or (2i, 2i+1) ("interleaved").  Dimensions at or above
    ``rotary_dim`` pass through.  The inverse frequencies are computed in float32 the way
    the reference builds its table (``1/powf(theta, d/head_size)``, rope_kernel.cu:69-94);
    the angle, sine and cosine are float32 in the kernel."""

    def __init__(self, theta: float, head_dim: int, dtype, device, rotary_dim: int = None,
                 pairing: str = "half"):
        rotary_dim = head_dim if rotary_dim is None else int(rotary_dim)
        if rotary_dim % 2 or not (0 < rotary_dim <= head_dim):
            raise ValueError(f"rotary_dim must be even and in (0, head_dim], got {rotary_dim}")
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"unknown rotary pairing {pairing!r}")
        self.theta, self.head_dim, self.rotary_dim, self.pairing = float(theta), head_dim, rotary_dim, pairing
        i = torch.arange(0, rotary_dim // 2, dtype=torch.float32)
        inv = 1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float32), (2.0 * i) / rotary_dim)
        self.inv_freq = inv.to(device)

    def kernel_args(self):
        return self.inv_freq, self.rotary_dim, self.pairing == "interleaved"


class NoPositionEncoding(PositionEncoding):
    def __init__(self, dtype=None, device=None, **_):
        pass

    def kernel_args(self):
        return None, 0, False


register_part("position", "rope", RotaryEncoding, replace=True)
register_part("position", "none", NoPositionEncoding, replace=True)
