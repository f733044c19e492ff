"""Interfaces of the parts a decoder is assembled from, and the registry that maps a
``PartSpec.kind`` to its class.

A part is constructed from its constants alone (sizes, eps, theta, window ...): it never
sees a model configuration and does not know which architecture it serves.  It states
which tensors it needs (``param_specs``), takes them (``load``) and computes
(``forward`` / ``add_norm``).  A new kind of part is added by subclassing one of these
classes and calling ``register_part``; nothing else in the package has to change.

Interfaces
----------
Norm:       ``add_norm(residual, delta, rows=None) -> normed``: residual += delta (float32,
            in place), then the normalised rows in the run dtype.
PositionEncoding: ``kernel_args() -> (inv_freq | None, rotary_dim, interleaved)`` for the
            mixer that applies it; one that brings its own code sets ``applies_itself`` and has
            ``apply(q, k, positions) -> (q, k)`` on float32 [rows, heads, head_dim] tensors
            (projection bias already added); its tensors live under the mixer's prefix + "position.".
            ``positions`` is int32 [rows]: the tokens' places in the sequence, or the position ids
            the step's entries brought (``StepEntry.position_ids``), then [rows, axes] when they
            have several axes.
Mixer:      ``cache_need() -> KVNeed | PagedNeed | StateNeed | None`` (what it keeps between steps) and
            ``forward(x, ctx, cache) -> y`` over all rows of the step.
FeedForward: ``forward(x, ctx) -> y``.
Block:      ``forward(residual, delta, ctx, cache) -> (residual, delta)``: the arrangement
            of norms, mixer and feed-forward; ``delta`` is the not-yet-added output of the
            previous part, so that the add is fused with the next norm.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch

from ..config.specs import ConfigError, PartSpec
from ..weights.loader import ParamSpec


@dataclass(frozen=True)
class CacheTensor:
    """One tensor of a paged cache layer: ``[page, heads, page_tokens, width]`` per layer."""
    name: str
    heads: int
    width: int


@dataclass(frozen=True)
class PagedNeed:
    """What a mixer keeps per token, in pages: any number of named tensors, each with its own
    heads and width (keys and values of different widths, one compressed latent, ...), and how
    long a token is kept (``window`` None: for ever; W: while one of the last W).  Layers with
    equal needs share a page pool and a block table."""
    tensors: Tuple[CacheTensor, ...]
    window: Optional[int] = None


@dataclass(frozen=True)
class KVNeed:
    """Keys and values of equal geometry in pages: the usual case of ``PagedNeed``."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None

    @property
    def tensors(self) -> Tuple[CacheTensor, ...]:
        return (CacheTensor("k", self.num_kv_heads, self.head_dim),
                CacheTensor("v", self.num_kv_heads, self.head_dim))


@dataclass(frozen=True)
class StateNeed:
    """A fixed-size state per request (one row per request slot).  The row of a request is
    zeroed by the step function before the request's first tokens run (also when a preempted
    request starts over), so a mixer finds zeros at ``context_before == 0``; it is never
    cleared otherwise, and what a mixer leaves there is what it finds at the request's next
    step.  One more row than there are request slots exists: the padding rows of a captured
    decode step point at it."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Part:
    def param_specs(self, prefix: str) -> List[ParamSpec]:
        return []

    def load(self, tensors: Dict[str, torch.Tensor], prefix: str) -> None:
        pass

    def kernel_libraries(self, dtype: torch.dtype):
        """(library, defines) pairs this part will launch, so they can be built together."""
        return []


class Norm(Part):
    def add_norm(self, residual, delta, rows=None, out_dtype=None):
        raise NotImplementedError


class PositionEncoding(Part):
    applies_itself = False      # True: the mixer calls apply() instead of handing kernel_args() to its kernel

    def kernel_args(self):
        raise NotImplementedError

    def apply(self, q, k, positions):
        raise NotImplementedError


class Mixer(Part):
    # Steps of single decoded tokens are captured once and replayed as CUDA graphs when every
    # mixer of the model sets this: it then steps such tokens with device tensors only (the
    # step's arrays, ``ctx.state_slots``), never with values read on the host, which a replay
    # would not see change.  A mixer that loops over the requests on the host leaves it False.
    decode_capturable = False

    def cache_need(self):
        return None

    def work_keys(self):
        """Attention work lists this mixer needs from the step: (heads per kv head,
        tile rows, window) triples."""
        return []

    def forward(self, x, ctx, cache):
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x, ctx):
        raise NotImplementedError


class Block(Part):
    mixer: Mixer

    def forward(self, residual, delta, ctx, cache):
        raise NotImplementedError


_PARTS: Dict[Tuple[str, str], Callable[..., Part]] = {}
CATEGORIES = ("norm", "position", "mixer", "feed_forward", "block")


def register_part(category: str, kind: str, factory: Callable[..., Part], replace: bool = False):
    if category not in CATEGORIES:
        raise ConfigError(f"unknown part category {category!r}; one of {CATEGORIES}")
    if (category, kind) in _PARTS and not replace:
        raise ConfigError(f"{category} part {kind!r} is already registered")
    _PARTS[(category, kind)] = factory


def build_block(spec, dtype: torch.dtype, device) -> Block:
    """A block from its ``BlockSpec``; ``spec.kind`` names the arrangement."""
    key = ("block", spec.kind)
    if key not in _PARTS:
        known = sorted(k for c, k in _PARTS if c == "block")
        raise ConfigError(f"no block arrangement {spec.kind!r}; known: {', '.join(known)}")
    return _PARTS[key](spec=spec, dtype=dtype, device=device)


def build_part(category: str, spec: PartSpec, dtype: torch.dtype, device) -> Part:
    key = (category, spec.kind)
    if key not in _PARTS:
        known = sorted(k for c, k in _PARTS if c == category)
        raise ConfigError(f"no {category} part of kind {spec.kind!r}; known: {', '.join(known)}")
    return _PARTS[key](dtype=dtype, device=device, **spec.args)
