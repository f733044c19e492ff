"""Architecture-neutral descriptions of what a model is made of.

A model is data: a list of block specifications (each naming its mixer, its
feed-forward, its norms and its position encoding, with every size and constant
as a field) and a run order (which block runs when, and into which cache layer).
The parts in ``parts/`` are built from these records; no part learns which
architecture it belongs to, and an architecture is only a function from its
``config.json`` to a ``ModelSpec``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """``kind`` selects the class in the part registry; ``args`` are its constants."""
    kind: str
    args: Dict[str, Any] = field(default_factory=dict)

    def __hash__(self):  # args is a dict: hash by its sorted items
        return hash((self.kind, tuple(sorted((k, repr(v)) for k, v in self.args.items()))))


@dataclass(frozen=True)
class BlockSpec:
    """One layer: how mixer, feed-forward and norms are arranged (``kind``), the
    parts themselves, and the prefix of its tensors in the checkpoint."""
    kind: str                      # arrangement, e.g. "prenorm"
    mixer: PartSpec
    feed_forward: PartSpec
    norm_mixer: PartSpec
    norm_feed_forward: PartSpec
    prefix: str                    # e.g. "model.layers.3."
    names: Dict[str, str] = field(default_factory=dict)  # sub-prefixes inside the block


@dataclass(frozen=True)
class RunStep:
    """One entry of the run order.

    ``block``: index into ``ModelSpec.blocks`` (a block may be named twice).
    ``cache_layer``: which cache layer this execution uses; two run steps that name
    the same cache layer share it.  ``writes_cache``: False lets a layer read the
    keys and values another layer wrote without writing its own.
    """
    block: int
    cache_layer: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    blocks: Tuple[BlockSpec, ...]
    run_order: Tuple[RunStep, ...]
    final_norm: PartSpec
    embedding_name: str
    final_norm_name: str
    lm_head_name: Optional[str]    # None: the head is the embedding table (tied)
    max_position: int
    eos_token_ids: Tuple[int, ...] = ()

    @property
    def num_cache_layers(self) -> int:
        return 1 + max((s.cache_layer for s in self.run_order), default=-1)


class ConfigError(ValueError):
    """A config.json that cannot describe a model this engine can run."""
