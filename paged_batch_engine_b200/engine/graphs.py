"""Decode steps as CUDA graphs.

A step in which every request brings exactly one token has the same launches every time;
only the integers the kernels read change.  Such steps are captured once per (batch
bucket, key-split bucket) with all integer arrays living in one persistent device buffer
at fixed offsets, and replayed after a single host-to-device copy of that buffer.  Rows
beyond the live requests are padding: they write nothing to the cache, carry idle
attention work items, and their logits are dropped.

Split boundaries lie at multiples of the step's split size, which follows from the number of
requests in the step (512 keys up to four requests, 256 beyond), and the fused decode kernel
picks its cluster size from the step's size too: a request's logits therefore agree between
a captured step, an eager step and steps of other sizes up to the rounding of float32 sums
taken in another order, not bit for bit.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import gc
import time
import weakref

import numpy as np
import torch

from ..cache.manager import decode_work_fill
from ..csrc import ops
from .batch import (AttentionWork, GroupArrays, StepContext, StepEntry,
                    attention_work_arrays, choose_split_keys)


def _bucket(n: int, cap: Optional[int] = None) -> int:
    b = 1
    while b < n:
        b *= 2
    return b if cap is None else min(b, max(cap, n))


def splits_bound(longest: int, window: Optional[int], split_keys: int) -> int:
    """The most key splits any request of at most ``longest`` tokens needs (see
    ``DecodeGraphs._splits_needed``)."""
    full = (longest + split_keys - 1) // split_keys
    if not window:
        return max(1, full)
    span = min(longest, int(window))
    return max(1, min(full, (span + split_keys - 2) // split_keys + 1))


def _batch_bucket(n: int) -> int:
    """Rows of the captured step that takes n requests: powers of two, and from 24 on also the
    sizes half-way (24, 48, 96 ...), so that padding rows cost the projections at most a third
    (33 requests in a step of 64 rows took 4.26 ms, 32 in their own 3.87)."""
    b = _bucket(n)
    return 3 * b // 4 if b >= 32 and n <= 3 * b // 4 else b


class DecodeStepContext(StepContext):
    """A StepContext whose arrays are fixed views of one persistent buffer."""
    captured = True               # its launches are recorded once and replayed

    def __init__(self, manager, device, work_keys, batch: int, splits: int, bt_strides: Sequence[int],
                 state_pad_slot: int = 0):
        self.manager, self.device = manager, device
        self.state_pad_slot = int(state_pad_slot)     # the state row that padding rows point at
        self.page_tokens = manager.page_tokens
        self.batch, self.splits = batch, splits
        self.split_keys = choose_split_keys(batch)
        self.num_tokens = self.num_requests = self.num_wanted = batch
        self.work_keys = list(work_keys)
        B, S = batch, splits
        off = 0
        lay: Dict[str, Tuple[int, Tuple[int, ...]]] = {}

        def place(name, shape):
            nonlocal off
            n = int(np.prod(shape))
            lay[name] = (off, tuple(shape))
            off += (n + 3) // 4 * 4
        for name in ("tokens", "positions", "q_start", "q_len", "seq_len", "want", "state"):
            place(name, (B,))
        for g, stride in enumerate(bt_strides):
            place(f"bt{g}", (B, stride))
            place(f"slots{g}", (B,))
        for i, _ in enumerate(self.work_keys):
            place(f"work{i}", (B * S, 4))
            place(f"tsr{i}", (B,))
            place(f"st{i}", (B,))
            place(f"sc{i}", (B,))
        self._layout, self._size = lay, off
        self.host = torch.zeros(off, dtype=torch.int32, pin_memory=True)
        self._host_np = self.host.numpy()
        self._views: Dict[str, np.ndarray] = {}
        self._handles: List[int] = []
        self._known = np.zeros((1, 0), dtype=np.int32)
        self._handles_np = np.zeros(0, dtype=np.int64)
        self._ctx = np.zeros(0, dtype=np.int64)
        self._arange = np.arange(B, dtype=np.int64)
        self._srange = np.arange(S, dtype=np.int64)
        self._ones = np.ones(B, dtype=np.int64)
        self.state_slots_host = np.zeros(0, dtype=np.int64)
        self.dev = torch.zeros(off, dtype=torch.int32, device=device)
        # set after every copy of the pinned buffer: the next fill rewrites that buffer and must
        # not start before the copy has read it (steps are launched ahead of one another)
        self._copied = torch.cuda.Event() if torch.device(device).type == "cuda" else None
        self._copy_pending = False

        def view(name):
            o, shape = lay[name]
            return self.dev[o:o + int(np.prod(shape))].view(shape)
        self.token_ids, self.positions = view("tokens"), view("positions")
        self.position_ids = self.positions          # captured steps take the places in the sequence
        self.q_start, self.q_len, self.seq_len = view("q_start"), view("q_len"), view("seq_len")
        self.want_rows, self.state_slots = view("want"), view("state")
        self._groups = [GroupArrays(view(f"bt{g}"), stride, view(f"slots{g}"))
                        for g, stride in enumerate(bt_strides)]
        self._h("q_start")[:] = np.arange(B)
        self._h("want")[:] = np.arange(B)
        for i, _ in enumerate(self.work_keys):
            self._h(f"tsr{i}")[:] = np.arange(B)
            self._h(f"st{i}")[:] = np.arange(B)
        self._work = {}
        for i, key in enumerate(self.work_keys):
            grp = self._groups[key[0]]
            self._work[key] = AttentionWork(
                q_start=self.q_start, q_len=self.q_len, seq_len=self.seq_len,
                block_table=grp.block_table, bt_stride=grp.bt_stride, work=view(f"work{i}"),
                num_work=B * S, tok_split_row=view(f"tsr{i}"), split_tokens=view(f"st{i}"),
                split_counts=view(f"sc{i}"), num_split_rows=B, max_splits=S, split_keys=self.split_keys,
                tile_rows=key[2], kinds=1 if key[1] <= 16 else 2,
                # a captured step serves split counts from half its capacity up to all of it
                small_items=(3 * B * S + 3) // 4, decode_rows=B, longest_keys=S * self.split_keys)

    def _h(self, name):
        v = self._views.get(name)
        if v is None:
            o, shape = self._layout[name]
            v = self._views[name] = self._host_np[o:o + int(np.prod(shape))].reshape(shape)
        return v

    def fill(self, entries: Sequence[StepEntry], vocab_size: int) -> None:
        """Writes this step's integers into the pinned buffer and copies it to the device.
        Rows keep their block tables between steps: when the same requests come back in the
        same order (the usual case while decoding), only newly added pages are written."""
        m, B, S, P = self.manager, self.batch, self.splits, self.page_tokens
        if self._copy_pending:
            self._copied.synchronize()        # almost always long satisfied
            self._copy_pending = False
        R = len(entries)
        handles = [e.handle for e in entries]
        same = handles == self._handles
        tokens = np.fromiter((e.tokens[0] for e in entries), dtype=np.int64, count=R)
        if tokens.min() < 0 or tokens.max() >= vocab_size:
            raise ValueError("a token id is outside the vocabulary")
        if not same:
            self._handles_np = np.asarray(handles, dtype=np.int64)
            self._known = np.zeros((max(len(m.groups), 1), R), dtype=np.int32)
            self._ctx = np.empty(R, dtype=np.int64)
            self.state_slots_host = np.empty(R, dtype=np.int64)
            for g in range(len(m.groups)):
                self._h(f"bt{g}")[:] = -1
                self._h(f"slots{g}")[:] = -1
        # context lengths, state slots, new block-table entries and cache slots in one call
        m.decode_fill(self._handles_np, self._ctx, self.state_slots_host,
                      [self._h(f"bt{g}") for g in range(len(m.groups))],
                      [self._h(f"slots{g}") for g in range(len(m.groups))], self._known, refresh=not same)
        ctx_before = self._ctx
        self.q_len_host = self._ones[:R]
        self.seq_len_host = ctx_before + 1
        self.q_start_host = self._arange[:R]
        self.context_before_host = ctx_before
        if not same:
            q = self._h("q_len"); q[:] = 0; q[:R] = 1
            st = self._h("state"); st[:] = self.state_pad_slot; st[:R] = self.state_slots_host
        for i, key in enumerate(self.work_keys):
            # positions, lengths, tokens (once) and the work list of this key, in the host library
            first = i == 0
            decode_work_fill(R, B, S, ctx_before, key[3], self.split_keys, self._h(f"work{i}"),
                             self._h(f"sc{i}"), self._h("positions") if first else None,
                             self._h("seq_len") if first else None, self._h("tokens") if first else None,
                             tokens if first else None, refresh=not same)
        if not self.work_keys:
            self._h("tokens")[:R] = tokens
            self._h("positions")[:R] = ctx_before
            self._h("seq_len")[:R] = ctx_before + 1
        self._handles = handles
        self.dev.copy_(self.host, non_blocking=True)
        if self._copied is not None:
            self._copied.record()
            self._copy_pending = True

    def attention_work(self, group, group_size, tile_rows, window, num_heads, head_dim):
        w = self._work[(group, group_size, tile_rows, window)]
        few = w.small_items * (num_heads // group_size) <= ops.decode_block_max_items(self.device)
        w.kinds = (w.kinds & ~4) | (4 if few else 0)
        if w.part_o is None:
            w.part_o = torch.empty((self.batch, num_heads, self.splits, head_dim), dtype=torch.float32,
                                   device=self.device)
            w.part_ml = torch.empty((self.batch, num_heads, self.splits, 2), dtype=torch.float32,
                                    device=self.device)
        return w


class DecodeGraphs:
    """Captured decode steps of one runner, keyed by (batch bucket, split bucket)."""

    def __init__(self, runner, max_context: int):
        # no reference cycle with the runner: an engine that goes out of use is freed at once,
        # not by a later garbage collection that might fall into another engine's capture
        self.runner = weakref.proxy(runner)
        self.max_context = int(max_context)
        self.graphs: Dict[Tuple[int, int], Tuple[torch.cuda.CUDAGraph, DecodeStepContext, torch.Tensor]] = {}
        self.replays = 0
        self.launches_per_replay = 0      # this package's kernels inside one captured step
        self.last_h2d_bytes = 0           # size of the integer buffer copied before a replay
        self.capture_seconds = 0.0        # host time spent capturing (warm-up run included)
        self._capture_stream = None

    def eligible(self, entries: Sequence[StepEntry]) -> bool:
        if not all(len(e.tokens) == 1 and list(e.want) == [0] and e.position_ids is None for e in entries):
            return False
        # a captured step is recorded once: a mixer that runs host logic per step (loops over the
        # requests, reads lengths on the host) cannot be in it; every mixer says which it is
        if not self.runner.model.decode_capturable():
            return False
        # one row tile per request is what a fixed work list holds
        return all(gsize <= tile_rows for _, gsize, tile_rows, _ in self.runner._work_keys)

    def _splits_needed(self, entries, split_keys: int) -> int:
        """Key splits a request of this step can need at most, from the longest request alone.
        Without a window that is the longest request's own count.  Under a window W a request
        of length n reads keys [max(0, n - W), n), and how many splits of ``split_keys`` that
        range touches depends on where it lies: a shorter request can touch one more than the
        longest.  A range of L keys touches at most (L + split_keys - 2) // split_keys + 1
        splits wherever it lies, so that bound (capped by the unwindowed count) holds for
        every request of the step and does not move as the requests grow."""
        m = self.runner.cache
        longest = m.max_reserved_len([e.handle for e in entries])
        return max([1] + [splits_bound(longest, window, split_keys)
                          for _, _, _, window in self.runner._work_keys])

    def run(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``device_tokens`` (int32 on the device, one per entry): the token ids of this step
        when the host does not know them yet (the step before is still running and they are
        what it samples); they replace the entries' placeholder ids on the device."""
        runner = self.runner
        R = len(entries)
        B = _batch_bucket(R)
        S = _bucket(self._splits_needed(entries, choose_split_keys(B)))
        key = (B, S)
        if key not in self.graphs:
            t0 = time.perf_counter()
            self.graphs[key] = self._capture(B, S, entries)
            self.capture_seconds += time.perf_counter() - t0
        graph, ctx, logits = self.graphs[key]
        ctx.fill(entries, runner.model.spec.vocab_size)
        self.last_h2d_bytes = ctx._size * 4
        if device_tokens is not None:
            ctx.token_ids[:R].copy_(device_tokens[:R], non_blocking=True)
        graph.replay()
        self.replays += 1
        return logits[:R]

    def _capture(self, B: int, S: int, entries):
        runner = self.runner
        P = runner.cache.page_tokens
        need = max(len(runner.cache.block_table(e.handle, g)) for e in entries
                   for g in range(len(runner.cache.groups))) if runner.cache.groups else 1
        cap = max((self.max_context + P - 1) // P, need, 1)
        strides = [cap for _ in runner.cache.groups]
        ctx = DecodeStepContext(runner.cache, runner.device, runner._work_keys, B, S, strides,
                                state_pad_slot=runner.storage.state_pad_slot)
        ctx.fill(entries, runner.model.spec.vocab_size)
        # Warm up on a side stream (library handles, lazy kernel loading), then capture.  The
        # warm-up and the capture write this step's keys and values to the slots the step
        # will write anyway, so the cache is not disturbed.
        # A mixer's state rows are not: the warm-up would step them once more than the step
        # itself (which runs when the captured graph is first replayed), so they are put back.
        kept = {layer: t.clone() for layer, t in runner.storage.state.items()}
        side = torch.cuda.Stream(device=runner.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            runner.model.forward(ctx, runner.storage)
        torch.cuda.current_stream().wait_stream(side)
        for layer, t in kept.items():
            runner.storage.state[layer].copy_(t)
        torch.cuda.synchronize()
        from ..csrc import ops
        before = ops.launch_count()
        graph = torch.cuda.CUDAGraph()
        # Destroying another engine's captured graphs (or pinned buffers) while this capture is
        # open would invalidate it: the collector stays off until the capture has ended.  The
        # capture is begun and ended by hand on a side stream: the library's context manager
        # would also run a full garbage collection and hand all cached device memory back to
        # the driver first, after which every buffer of the next steps is allocated anew
        # (a capture took 40 to 60 ms that way, most of it outside the capture itself).
        gc_was_on = gc.isenabled()
        gc.disable()
        cap_stream = self._capture_stream
        if cap_stream is None:
            cap_stream = self._capture_stream = torch.cuda.Stream(device=runner.device)
        cap_stream.wait_stream(torch.cuda.current_stream())
        try:
            with torch.cuda.stream(cap_stream):
                graph.capture_begin()
                try:
                    logits = runner.model.forward(ctx, runner.storage)
                finally:
                    graph.capture_end()
        finally:
            if gc_was_on:
                gc.enable()
        torch.cuda.current_stream().wait_stream(cap_stream)
        self.launches_per_replay = ops.launch_count() - before
        return graph, ctx, logits
