"""The step function: a model, its cache, and ``step(entries) -> logits``.

``step`` runs only the tokens it is given, as one batch, against the cache that earlier
steps left, and returns float32 logits at the wanted places.  It allocates no pages and
frees none: the caller reserves a request's tokens before the step
(``cache.reserve``); the step marks them computed afterwards (``cache.commit``), which
is also when a windowed layer group gives back pages the window has passed.

The reference's step is ``Qwen2Model::forward_mixed_batch``
(infMain/source/model/qwen2_batch.cpp:473-805), which also reserves prompt pages,
computes logits for every row and synchronises before committing.
"""
from __future__ import annotations

import os
from typing import List, Optional, Sequence

import torch

from ..cache.storage import CacheStorage
from ..config.registry import load_config
from ..models.decoder import DecoderModel
from ..weights.loader import load_weights
from ..weights.random_init import random_tensor
from .batch import StepContext, StepEntry


def _parse_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        return dtype
    table = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
             "fp32": torch.float32}
    if dtype not in table:
        raise ValueError(f"dtype must be bfloat16 or float32, got {dtype!r}")
    return table[dtype]


def require_cuda(device) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda":
        raise RuntimeError("this engine runs on CUDA devices only; there is no CPU path")
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device is available: the engine cannot run")
    return device


def build_model(config, dtype, device) -> DecoderModel:
    """config: a folder, a config.json path, a dict or a typed config with model_spec()."""
    if hasattr(config, "model_spec"):
        arch_builder, typed = None, config
    else:
        arch, typed = load_config(config)
        arch_builder = arch.builder
    spec = typed.model_spec()
    if arch_builder is not None:
        return arch_builder(spec, dtype, device)
    return DecoderModel(spec, dtype, device)


class ModelRunner:
    def __init__(self, model: DecoderModel, page_tokens: int = 16, num_pages=None,
                 max_requests: int = 256, max_cache_tokens: Optional[int] = None, lifo: bool = False,
                 poison: bool = False, max_context: Optional[int] = None):
        self.model = model
        self.device = model.device
        if num_pages is None:
            if max_cache_tokens is None:
                raise ValueError("give num_pages or max_cache_tokens")
            num_pages = (max_cache_tokens + page_tokens - 1) // page_tokens
        self.storage = CacheStorage(model.cache_needs, page_tokens, num_pages, max_requests,
                                    model.dtype, self.device, lifo=lifo, poison=poison)
        self.cache = self.storage.manager
        self._work_keys = model.work_keys(self.storage)
        self.steps_run = 0
        self.graphs = None
        if self.device.type == "cuda":
            from .graphs import DecodeGraphs
            cap = self.cache.capacity_tokens()
            self.graphs = DecodeGraphs(self, min(max_context or model.spec.max_position, cap))

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_folder(cls, folder: str, dtype="bfloat16", device="cuda:0", **kw) -> "ModelRunner":
        device = require_cuda(device)
        dtype = _parse_dtype(dtype)
        model = build_model(folder, dtype, device)
        model.build_kernels()
        model.load(load_weights(folder, model.param_specs(), dtype, device))
        return cls(model, **kw)

    @classmethod
    def from_random(cls, config, seed: int = 0, dtype="bfloat16", device="cuda:0", **kw) -> "ModelRunner":
        """Random weights made on the device (for measurements; no folder is written)."""
        device = require_cuda(device)
        dtype = _parse_dtype(dtype)
        model = build_model(config, dtype, device)
        model.build_kernels()
        tensors = {}
        for p in model.param_specs():
            if p.optional:
                continue
            tensors[p.name] = random_tensor(p, seed, dtype, device=device)
        model.load(tensors)
        return cls(model, **kw)

    # ------------------------------------------------------------------ the step
    def step(self, entries: Sequence[StepEntry], commit: bool = True,
             decode_graph: bool = False, device_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Runs the entries as one batch; float32 logits [wanted, vocab] on the device.
        ``decode_graph``: replay a captured CUDA graph when every entry is a single token.
        ``device_tokens``: the step's token ids as an int32 device tensor (a step scheduled
        ahead of the one that samples them); captured decode steps only."""
        if self.storage.state:
            # a request whose first tokens run now finds its state rows zeroed (a new request, or
            # one that starts over after a preemption); see parts.StateNeed
            self.storage.zero_state([self.cache.state_slot(e.handle) for e in entries
                                     if self.cache.context_len(e.handle) == 0])
        if decode_graph and self.graphs is not None and self.graphs.eligible(entries):
            logits = self.graphs.run(entries, device_tokens)
        elif device_tokens is not None:
            raise ValueError("token ids on the device are taken by captured decode steps only")
        else:
            ctx = StepContext(self.cache, entries, self.device, self._work_keys,
                              vocab_size=self.model.spec.vocab_size)
            logits = self.model.forward(ctx, self.storage)
        if commit:
            for e in entries:
                self.cache.commit(e.handle, len(e.tokens))
        self.steps_run += 1
        return logits
