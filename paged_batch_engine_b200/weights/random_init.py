"""Seeded random weights: a model folder (config.json + model.safetensors) from a
configuration and a seed, or tensors made straight on the device for measurements.

Distributions: matrices N(0, 0.02) as the reference's Python initialiser does
(tools/model_qwen2.py:242-248), q/k/v biases N(0, 0.02) and norm gains 1 + N(0, 0.1) so
that no bias or gain is a silent identity in a test.  Each tensor has its own generator
seeded from (seed, tensor name): adding or reordering tensors does not change the others.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Sequence

import torch

from .loader import ParamSpec
from .safetensors_io import save_file


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def _distribution(name: str, shape):
    if len(shape) <= 1:
        if name.endswith("bias"):
            return 0.0, 0.02
        return 1.0, 0.1      # gains
    return 0.0, 0.02


def random_tensor(spec: ParamSpec, seed: int, dtype: torch.dtype, device="cpu",
                  scale: float = 1.0) -> torch.Tensor:
    if spec.kind == "int":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    g = torch.Generator(device=device)
    g.manual_seed(_tensor_seed(seed, spec.name))
    mean, std = _distribution(spec.name, spec.shape)
    t = torch.empty(spec.shape, dtype=torch.float32 if len(spec.shape) <= 1 else dtype, device=device)
    if t.numel():
        t.normal_(mean, std * scale, generator=g)
    return t


def random_state_dict(params: Sequence[ParamSpec], seed: int, dtype: torch.dtype,
                      device="cpu") -> Dict[str, torch.Tensor]:
    return {p.name: random_tensor(p, seed, dtype, device) for p in params if not p.optional}


def write_random_model(folder: str, config, params: Sequence[ParamSpec], seed: int,
                       dtype: torch.dtype = torch.bfloat16) -> str:
    """Write ``config.json`` and ``model.safetensors`` with seeded random weights."""
    os.makedirs(folder, exist_ok=True)
    d = config.to_dict() if hasattr(config, "to_dict") else dict(config)
    d["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32",
                        torch.float16: "float16"}[dtype]
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(d, f, indent=2, sort_keys=True)
    tensors = {}
    for p in params:
        if p.optional:
            continue
        t = random_tensor(p, seed, torch.float32)
        tensors[p.name] = t.to(dtype) if p.kind == "float" else t
    save_file(tensors, os.path.join(folder, "model.safetensors"),
              metadata={"format": "pt", "seed": str(seed)})
    return folder
