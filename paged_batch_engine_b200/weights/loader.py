"""Weights by tensor name.

The reference reads a position-addressed ``.bin`` (tools/export_qwen2.py:170-198; reader
infMain/source/model/qwen2.cpp:793-945) in which a wrong shape cannot be noticed.  Here a
model states the tensors it needs (name, shape) and the loader answers with the tensors or
with ONE error that lists everything missing, unexpected and mis-shaped.

dtype rule: floating tensors stored in 16 bits are kept in bfloat16 for a bfloat16 run,
integer tables become int32, and a tensor stored in 32 bits stays in 32 bits; a float32
run upcasts every floating tensor exactly.  One-dimensional parameters (norm gains,
biases) are always held in float32: the upcast is exact and the kernels read them once.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from .safetensors_io import SafetensorsError, open_model_files


@dataclass(frozen=True)
class ParamSpec:
    name: str
    shape: Tuple[int, ...]
    kind: str = "float"      # "float" or "int"
    optional: bool = False   # read if present, never reported as missing or unexpected


class WeightsError(ValueError):
    def __init__(self, message, missing=(), unexpected=(), wrong_shape=(), wrong_dtype=()):
        super().__init__(message)
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)


_FLOAT = ("F32", "BF16", "F16")
_INT = ("I64", "I32", "I16", "I8", "U8")


def target_dtype(stored: str, kind: str, ndim: int, run_dtype: torch.dtype) -> torch.dtype:
    if kind == "int":
        return torch.int32
    if run_dtype == torch.float32 or ndim <= 1 or stored == "F32":
        return torch.float32
    return torch.bfloat16


def check_names(expected: Sequence[ParamSpec], present: Dict[str, Tuple[str, Tuple[int, ...]]],
                where: str) -> None:
    exp = {p.name: p for p in expected}
    missing = sorted(n for n, p in exp.items() if n not in present and not p.optional)
    unexpected = sorted(n for n in present if n not in exp)
    wrong_shape, wrong_dtype = [], []
    for n, p in exp.items():
        if n not in present:
            continue
        dt, shape = present[n]
        if tuple(shape) != tuple(p.shape):
            wrong_shape.append((n, tuple(shape), tuple(p.shape)))
        ok = _INT if p.kind == "int" else _FLOAT
        if dt not in ok:
            wrong_dtype.append((n, dt, "/".join(ok)))
    if missing or unexpected or wrong_shape or wrong_dtype:
        lines = [f"weights in {where} do not match the model:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"  wrong shape ({len(wrong_shape)}): " + "; ".join(
                f"{n} is {list(s)}, expected {list(e)}" for n, s, e in sorted(wrong_shape)))
        if wrong_dtype:
            lines.append(f"  wrong dtype ({len(wrong_dtype)}): " + "; ".join(
                f"{n} is {d}, expected one of {e}" for n, d, e in sorted(wrong_dtype)))
        raise WeightsError("\n".join(lines), missing, unexpected, wrong_shape, wrong_dtype)


def load_weights(folder: str, expected: Sequence[ParamSpec], run_dtype: torch.dtype,
                 device) -> Dict[str, torch.Tensor]:
    """Read the expected tensors of a model folder onto ``device``."""
    try:
        files = open_model_files(folder)
    except (SafetensorsError, OSError) as e:
        raise WeightsError(str(e)) from e
    present: Dict[str, Tuple[str, Tuple[int, ...]]] = {}
    owner = {}
    duplicates = []
    for f in files:
        for n, e in f.entries.items():
            if n in present:
                duplicates.append(n)
            present[n] = e
            owner[n] = f
    if duplicates:
        raise WeightsError(f"weights in {folder}: tensors stored twice: {', '.join(sorted(duplicates))}")
    check_names(expected, present, folder)
    out: Dict[str, torch.Tensor] = {}
    for p in expected:
        if p.name not in present:
            continue
        stored, _ = present[p.name]
        t = owner[p.name].tensor(p.name)
        out[p.name] = t.to(device=device, dtype=target_dtype(stored, p.kind, len(p.shape), run_dtype))
    for f in files:
        f.close()
    return out
