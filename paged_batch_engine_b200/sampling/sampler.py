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

    def __init__(self, device, max_requests: int = 0):
        self.device = device
        self._async_slots = []
        self._async_next = 0
        # the repetition penalty's table of seen tokens: a row of bytes per tracked request, made
        # when the first request with a penalty arrives
        self._seen = None
        self._seen_rows = max(int(max_requests), 8)
        self._slot_of = {}
        self._free_slots: List[int] = []

    # ------------------------------------------------------------------ seen tokens, on the device
    def tracked(self, key) -> bool:
        return key in self._slot_of

    def track(self, key, tokens: Sequence[int], vocab: int) -> None:
        """Starts a row of seen tokens for request ``key`` with the tokens it has so far; from
        then on every token sampled for it is marked on the device, so that the penalty needs
        nothing from the host."""
        if key in self._slot_of:
            return
        if self._seen is None or self._seen.shape[1] < vocab:
            ld = (vocab + 15) // 16 * 16
            self._seen = torch.zeros((self._seen_rows, ld), dtype=torch.uint8, device=self.device)
            self._free_slots = list(range(self._seen_rows - 1, -1, -1))
            self._slot_of = {}
        if not self._free_slots:
            more = torch.zeros_like(self._seen)
            self._free_slots = list(range(2 * self._seen_rows - 1, self._seen_rows - 1, -1))
            self._seen = torch.cat([self._seen, more])
            self._seen_rows *= 2
        slot = self._free_slots.pop()
        self._slot_of[key] = slot
        self._seen[slot].zero_()
        if len(tokens):
            ids = torch.from_numpy(np.asarray(tokens, dtype=np.int32)).to(self.device)
            ops.seen_mark(self._seen, ids, None, slot)

    def untrack(self, key) -> None:
        slot = self._slot_of.pop(key, None)
        if slot is not None:
            self._free_slots.append(slot)

    def _penalty_rows(self, params: Sequence[SamplingParams], keys):
        """(slots, penalties) on the device for the rows of a step, or None when no row has a
        tracked request with a penalty."""
        if keys is None or self._seen is None:
            return None
        slots = [self._slot_of.get(k, -1) if p.repetition_penalty != 1.0 else -1 for p, k in zip(params, keys)]
        if all(s < 0 for s in slots):
            return None
        pack = np.array([slots, [0] * len(slots)], dtype=np.int32)
        pack[1] = np.array([p.repetition_penalty for p in params], dtype=np.float32).view(np.int32)
        dev = torch.from_numpy(pack).to(self.device)
        return dev[0], dev[1].view(torch.float32)

    def sample_async(self, logits: torch.Tensor, params: Sequence[SamplingParams], counters: Sequence[int],
                     keys=None):
        """Launches the sampling of every row and the copy of the ids to pinned host memory;
        returns (ids on the device, ids on the host, event): the host list is valid once the
        event has completed, and holds one element more than there are rows: the kernels' status
        word (``ops.collect_status``), which ``read_async`` checks.  ``keys``: the rows' request keys; a row with a repetition penalty
        must belong to a tracked request (``track``).  Nothing here waits for the device: the
        rows' parameters go up from pinned memory (a copy from pageable memory would first wait
        for the stream, i.e. for the step that is still running).  Buffers rotate over four steps."""
        n = logits.shape[0]
        if any(p.repetition_penalty != 1.0 and (keys is None or not self.tracked(k))
               for p, k in zip(params, keys if keys is not None else [None] * n)):
            raise ValueError("sample_async: a row with a repetition penalty needs a tracked request")
        slot = self._async_slots[self._async_next % len(self._async_slots)] if self._async_slots else None
        if slot is None or slot[0].numel() < n + 1:
            cap = max(64, 2 * n)
            self._async_slots = [(torch.empty(cap, dtype=torch.int32, device=self.device),
                                  torch.empty(cap, dtype=torch.int32, pin_memory=True),
                                  torch.cuda.Event(),
                                  torch.empty((6, cap), dtype=torch.int32, device=self.device),
                                  torch.empty((6, cap), dtype=torch.int32, pin_memory=True)) for _ in range(4)]
            slot = self._async_slots[0]
            self._async_next = 0
        self._async_next += 1
        dev, host, event, pdev, phost = slot
        if all(p.is_greedy for p in params):
            ops.argmax(logits, dev[:n])
        else:
            # rows of the parameter block: temperature, top_p, uniform (float32 bits), top_k, the
            # penalty's slot of seen tokens (-1: none), the penalty (float32 bits)
            event.synchronize()              # the copy that last read this pinned block is over (four steps ago)
            block = phost.numpy()
            fl = block.view(np.float32)
            fl[0, :n] = [p.temperature for p in params]
            fl[1, :n] = [p.top_p for p in params]
            fl[2, :n] = [request_sample_uniform(p.seed, c) for p, c in zip(params, counters)]
            block[3, :n] = [p.top_k for p in params]
            slots = [self._slot_of.get(k, -1) if p.repetition_penalty != 1.0 else -1
                     for p, k in zip(params, keys if keys is not None else [None] * n)]
            block[4, :n] = slots
            fl[5, :n] = [p.repetition_penalty for p in params]
            pdev[:, :n].copy_(phost[:, :n], non_blocking=True)
            fdev = pdev.view(torch.float32)
            penalised = any(sl >= 0 for sl in slots)
            if penalised:
                ops.penalty_seen(logits, self._seen, pdev[4, :n], fdev[5, :n])
            ops.sample(logits, fdev[0, :n], pdev[3, :n], fdev[1, :n], fdev[2, :n], out=dev[:n])
            if penalised:
                ops.seen_mark(self._seen, dev[:n], pdev[4, :n])
        ops.collect_status(dev[n:n + 1])
        host[:n + 1].copy_(dev[:n + 1], non_blocking=True)
        event.record()
        return dev[:n], host[:n + 1], event

    def read_async(self, host: torch.Tensor, event) -> List[int]:
        """Waits for a ``sample_async`` and returns its ids; raises ``ops.KernelError`` when a
        kernel of the step reported a bounded wait that ran out (its ids are not valid)."""
        event.synchronize()
        vals = host.tolist()
        if vals[-1]:
            raise ops.KernelError(ops.status_message(self.device, vals[-1]))
        return vals[:-1]

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], counters: Sequence[int],
               seen: Sequence[Sequence[int]] = (), keys=None) -> List[int]:
        """The rows' tokens, on the host.  The repetition penalty takes its tokens from the
        tracked requests' table on the device (``keys``: the rows' request keys), or, without
        keys, from ``seen`` (a list of token lists, one per row)."""
        n = logits.shape[0]
        if n == 0:
            return []
        if all(p.is_greedy for p in params):
            return self._checked(ops.argmax(logits))
        pen = self._penalty_rows(params, keys)
        if pen is not None:
            ops.penalty_seen(logits, self._seen, pen[0], pen[1])
        elif keys is None:
            pen_rows, pen_tokens, pen_vals = [], [], []
            for r, p in enumerate(params):
                if p.repetition_penalty != 1.0 and r < len(seen):
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
        if pen is not None:
            ops.seen_mark(self._seen, out, pen[0])
        return self._checked(out)

    def _checked(self, ids: torch.Tensor) -> List[int]:
        """The ids on the host, with the kernels' status word read in the same transfer."""
        n = ids.numel()
        both = torch.empty(n + 1, dtype=torch.int32, device=ids.device)
        both[:n].copy_(ids)
        ops.collect_status(both[n:])
        vals = both.cpu().tolist()
        if vals[-1]:
            raise ops.KernelError(ops.status_message(self.device, vals[-1]))
        return vals[:-1]
