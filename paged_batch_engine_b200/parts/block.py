"""Arrangements of norms, mixer and feed-forward in a layer."""
from __future__ import annotations

from ..config.specs import BlockSpec
from .base import Block, build_part, register_part


class PreNormBlock(Block):
    """x -> norm -> mixer -> +x -> norm -> feed-forward -> +x  (reference:
    infMain/source/model/qwen2_batch.cpp:600-601, 753-759, 780).  Each add is carried as
    ``delta`` into the next norm so that add and norm are one kernel."""

    def __init__(self, spec: BlockSpec, dtype, device):
        self.spec = spec
        self.prefix = spec.prefix
        n = spec.names
        self.p_mixer = self.prefix + n.get("mixer", "mixer.")
        self.p_ffn = self.prefix + n.get("feed_forward", "feed_forward.")
        self.p_norm1 = self.prefix + n.get("norm_mixer", "norm_mixer.")
        self.p_norm2 = self.prefix + n.get("norm_feed_forward", "norm_feed_forward.")
        self.norm1 = build_part("norm", spec.norm_mixer, dtype, device)
        self.mixer = build_part("mixer", spec.mixer, dtype, device)
        self.norm2 = build_part("norm", spec.norm_feed_forward, dtype, device)
        self.ffn = build_part("feed_forward", spec.feed_forward, dtype, device)

    def parts(self):
        return [(self.norm1, self.p_norm1), (self.mixer, self.p_mixer), (self.norm2, self.p_norm2),
                (self.ffn, self.p_ffn)]

    def param_specs(self, prefix=""):
        out = []
        for part, p in self.parts():
            out += part.param_specs(p)
        return out

    def load(self, tensors, prefix=""):
        for part, p in self.parts():
            part.load(tensors, p)

    def kernel_libraries(self, dtype):
        out = []
        for part, _ in self.parts():
            out += part.kernel_libraries(dtype)
        return out

    def forward(self, residual, delta, ctx, cache):
        h = self.norm1.add_norm(residual, delta)
        a = self.mixer.forward(h, ctx, cache)
        f = self.norm2.add_norm(residual, a)
        m = self.ffn.forward(f, ctx)
        return residual, m


register_part("block", "prenorm", lambda spec, dtype, device: PreNormBlock(spec, dtype, device),
              replace=True)
