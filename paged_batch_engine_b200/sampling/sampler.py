"""Turns the step's logits into one token per sampled row, on the device."""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch

from ..csrc import ops
from .params import SamplingParams, request_sample_uniform


class Sampler:
    """All rows greedy: one argmax launch.  Otherwise an optional repetition-penalty launch
    and one sampling launch with per-row temperature, top_k, top_p and the request's own
    uniform draw; greedy rows inside such a batch take the argmax branch of the same
    kernel.  The reference sends every batch with top_k outside 1..32 or with a penalty
    through the host with the whole logits matrix (infMain/source/model/qwen2.cpp:1870-1987)."""

    def __init__(self, device):
        self.device = device
        self._async_slots = []
        self._async_next = 0

    def sample_async(self, logits: torch.Tensor, params: Sequence[SamplingParams], counters: Sequence[int]):
        """Launches the sampling of every row and the copy of the ids to pinned host memory;
        returns (ids on the device, ids on the host, event): the host list is valid once the
        event has completed.  No row may ask for a repetition penalty (that needs the request's
        tokens on the host).  Buffers rotate over four steps."""
        n = logits.shape[0]
        if any(p.repetition_penalty != 1.0 for p in params):
            raise ValueError("sample_async does not take a repetition penalty")
        slot = self._async_slots[self._async_next % len(self._async_slots)] if self._async_slots else None
        if slot is None or slot[0].numel() < n:
            cap = max(64, 2 * n)
            self._async_slots = [(torch.empty(cap, dtype=torch.int32, device=self.device),
                                  torch.empty(cap, dtype=torch.int32, pin_memory=True),
                                  torch.cuda.Event()) for _ in range(4)]
            slot = self._async_slots[0]
            self._async_next = 0
        self._async_next += 1
        dev, host, event = slot
        if all(p.is_greedy for p in params):
            ops.argmax(logits, dev[:n])
        else:
            floats = np.array([[p.temperature for p in params], [p.top_p for p in params],
                               [request_sample_uniform(p.seed, c) for p, c in zip(params, counters)]],
                              dtype=np.float32)
            fdev = torch.from_numpy(floats).to(self.device)
            kdev = torch.tensor([p.top_k for p in params], dtype=torch.int32, device=self.device)
            ops.sample(logits, fdev[0].contiguous(), kdev, fdev[1].contiguous(), fdev[2].contiguous(), out=dev[:n])
        host[:n].copy_(dev[:n], non_blocking=True)
        event.record()
        return dev[:n], host[:n], event

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], counters: Sequence[int],
               seen: Sequence[Sequence[int]]) -> List[int]:
        n = logits.shape[0]
        if n == 0:
            return []
        if all(p.is_greedy for p in params):
            return ops.argmax(logits).cpu().tolist()
        pen_rows, pen_tokens, pen_vals = [], [], []
        for r, p in enumerate(params):
            if p.repetition_penalty != 1.0:
                uniq = sorted(set(int(t) for t in seen[r]))
                pen_rows += [r] * len(uniq)
                pen_tokens += uniq
                pen_vals += [p.repetition_penalty] * len(uniq)
        if pen_rows:
            pack = np.array([pen_rows, pen_tokens], dtype=np.int32)
            dev = torch.from_numpy(pack).to(self.device)
            ops.apply_penalty(logits, dev[0].contiguous(), dev[1].contiguous(),
                              torch.tensor(pen_vals, dtype=torch.float32, device=self.device))
        floats = np.array([[p.temperature for p in params], [p.top_p for p in params],
                           [request_sample_uniform(p.seed, c) for p, c in zip(params, counters)]],
                          dtype=np.float32)
        fdev = torch.from_numpy(floats).to(self.device)
        kdev = torch.tensor([p.top_k for p in params], dtype=torch.int32, device=self.device)
        out = ops.sample(logits, fdev[0].contiguous(), kdev, fdev[1].contiguous(), fdev[2].contiguous())
        return out.cpu().tolist()
