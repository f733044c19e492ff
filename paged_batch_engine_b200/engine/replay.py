"""Trace replay: given token ids, step by step, through the engine's own step function.

A trace is a sequence of records ``{"step": s, "entries": [{"id", "tokens", "want"}],
"end": [ids]}``.  Each record's entries are one batch; a request's pages are reserved
before its tokens run and everything it holds is given back when it is named in ``end``.
Nothing is sampled.
"""
from __future__ import annotations

import json
import os
from typing import Callable, Dict, Iterable, Optional

import numpy as np
import torch

from ..csrc import ops
from .batch import StepEntry
from .runner import ModelRunner


class ReplayError(RuntimeError):
    pass


class TraceReplayer:
    """``decode_graphs``: steps in which every entry is one token whose logits are wanted go
    through the captured decode step (a replayed CUDA graph, as generation runs them) instead
    of the eager step.  ``device_tokens``: such steps also get their token ids the way a step
    launched ahead gets them, as a tensor on the device, with placeholder ids in the entries."""

    def __init__(self, runner: ModelRunner, decode_graphs: bool = False, device_tokens: bool = False):
        self.runner = runner
        self.handles: Dict[object, int] = {}
        self.decode_graphs = bool(decode_graphs)
        self.device_tokens = bool(device_tokens and decode_graphs)
        self.graph_steps = 0

    def _step(self, entries):
        graphs = self.runner.graphs
        if self.decode_graphs and graphs is not None and graphs.eligible(entries):
            self.graph_steps += 1
            if self.device_tokens:
                ids = torch.tensor([e.tokens[0] for e in entries], dtype=torch.int32).to(self.runner.device)
                entries = [StepEntry(e.handle, [0], e.want) for e in entries]
                return self.runner.step(entries, decode_graph=True, device_tokens=ids)
            return self.runner.step(entries, decode_graph=True)
        return self.runner.step(entries)

    def run_record(self, rec: dict) -> Optional[torch.Tensor]:
        """Runs one step; returns float32 logits [wanted, vocab] on the device, or None
        when the step wants none."""
        cache = self.runner.cache
        step = rec.get("step")
        entries = []
        for e in rec.get("entries", []):
            rid = e["id"]
            if rid not in self.handles:
                h = cache.add_request(rid)
                if h is None:
                    raise ReplayError(f"step {step}: no free request slot for {rid!r}")
                self.handles[rid] = h
            h = self.handles[rid]
            tokens = [int(t) for t in e["tokens"]]
            if not cache.reserve(h, len(tokens)):
                raise ReplayError(f"step {step}: the cache pool cannot hold {len(tokens)} more tokens "
                                  f"of request {rid!r}")
            entries.append(StepEntry(h, tokens, [int(w) for w in e.get("want", [])]))
        logits = None
        if entries:
            out = self._step(entries)
            ops.raise_on_kernel_status(self.runner.device)    # a wait that ran out is an error, not logits
            if out.shape[0] > 0:
                logits = out
        for rid in rec.get("end", []):
            if rid in self.handles:
                cache.free(self.handles.pop(rid))
        return logits


def replay_stream(runner: ModelRunner, lines: Iterable[str], out_dir: str,
                  report: Callable[[str], None], decode_graphs: bool = False) -> None:
    """Reads records line by line, writes ``<out_dir>/<step>.f32`` for steps that want
    logits and reports ``done <step>`` after each."""
    os.makedirs(out_dir, exist_ok=True)
    rp = TraceReplayer(runner, decode_graphs=decode_graphs)
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        logits = rp.run_record(rec)
        if logits is not None:
            arr = logits.detach().to("cpu", torch.float32).contiguous().numpy().astype("<f4", copy=False)
            with open(os.path.join(out_dir, f"{rec['step']}.f32"), "wb") as f:
                f.write(arr.tobytes())
        else:
            torch.cuda.synchronize()
        report(f"done {rec['step']}")
