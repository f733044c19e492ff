"""One step's batch as device arrays.

A step is a list of (request, its next tokens, the places whose logits are wanted).  The
rows of all requests are laid end to end; a row's position is the request's context
length before the step plus its offset.  This module turns that list into the integer
arrays the kernels read (positions, cache slots, block tables, request extents, and the
attention work lists), packs them into one pinned host buffer and copies them with one
transfer.

The reference builds the same kind of metadata in ``MixedBatchBuilder``
(infMain/source/serving/mixed_batch_builder.cpp:100-223: token_ids, positions, seq_lens,
block_tables padded with -1, logits_indices) and expands it per row in
``build_row_attention_metadata`` (infMain/source/model/qwen2_batch.cpp:304-469).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..csrc import ops

from ..cache.manager import CacheManager

SPLIT_KEYS = 256          # keys per split of a short request's long key range, many requests
SPLIT_KEYS_FEW = 512      # the same in steps of at most FEW_REQUESTS requests
FEW_REQUESTS = 4          # (a bucket edge of the captured decode steps)
MAX_SPLIT_TILES = 4       # requests with more row tiles than this are never split


def choose_split_keys(num_requests: int) -> int:
    """Keys per split for a step, by the number of its requests alone.  With one to four
    requests, splits are there to spread a long context over the multiprocessors, and a work
    item of 512 keys amortises its start-up better (one request with 32,768 keys: 50 -> 36 us a
    layer); with more requests, 256 keys keep the items even."""
    return SPLIT_KEYS_FEW if num_requests <= FEW_REQUESTS else SPLIT_KEYS


# Steps with at most this many requests run decoded tokens through the block-cooperative
# instance of the attention kernel (four warps share each key tile: shortest latency per work
# item); larger steps through the persistent warp-private instance (most bytes in flight).


@dataclass
class StepEntry:
    handle: int                 # the cache manager's request handle
    tokens: Sequence[int]       # the request's next tokens
    want: Sequence[int] = ()    # offsets among these tokens whose logits are wanted
    # Position ids of these tokens for the position encoding, when they are not the tokens'
    # places in the sequence: one integer per token, or a row of integers per token (an
    # encoding with several axes).  None: the place in the sequence.  Where a token lies in the
    # cache and what it may attend to always follow from its place in the sequence.
    position_ids: Optional[Sequence] = None


@dataclass
class GroupArrays:
    block_table: torch.Tensor   # int32 [R, stride]
    bt_stride: int
    slots: torch.Tensor         # int32 [T]


@dataclass
class AttentionWork:
    """Device arrays of one attention work list (see ``build_attention_work``)."""
    q_start: torch.Tensor
    q_len: torch.Tensor
    seq_len: torch.Tensor
    block_table: torch.Tensor
    bt_stride: int
    work: torch.Tensor
    num_work: int
    tok_split_row: torch.Tensor
    split_tokens: Optional[torch.Tensor]
    split_counts: Optional[torch.Tensor]
    num_split_rows: int
    max_splits: int
    split_keys: int
    tile_rows: int
    part_o: Optional[torch.Tensor] = None
    part_ml: Optional[torch.Tensor] = None
    kinds: int = 0                  # bit 0: row tiles of at most 16 packed rows exist, bit 1: larger ones,
    #                                 bit 2: few enough of the small ones for the block-cooperative instance
    small_items: int = 0            # live work items with at most 16 packed rows
    decode_rows: int = 0            # rows of a step of decoded tokens only (0: the step has prompt portions)
    longest_keys: int = 0           # the longest context of the step (a captured step: of its capacity)


def attention_work_arrays(q_len: np.ndarray, seq_len: np.ndarray, q_start: np.ndarray,
                          group_size: int, tile_rows: int, window: Optional[int],
                          split_keys: int = SPLIT_KEYS, force_split: bool = False,
                          fixed_splits: int = 0):
    """Host arrays of an attention work list.

    Each request's rows are packed with the ``group_size`` query heads of a key/value head
    (packed = row * group_size + head) and cut into tiles of ``tile_rows``.  A request with
    few tiles and a long key range is also cut along its keys into splits of
    ``split_keys``, at absolute multiples of ``split_keys``; the number of splits follows
    from the request's own lengths only.  Returns (work [n,4], tok_split_row [T],
    split_tokens, split_counts, max_splits).  ``force_split`` lists every row as a split
    row and ``fixed_splits`` pads every request to that many work items (idle ones carry
    request -1), which gives a work list of fixed size for a captured graph.
    """
    R = len(q_len)
    q_len = q_len.astype(np.int64)
    seq_len = seq_len.astype(np.int64)
    packed = q_len * group_size
    m_tiles = (packed + tile_rows - 1) // tile_rows
    pos0 = seq_len - q_len
    lo_req = np.maximum(0, pos0 - window + 1) if window else np.zeros(R, dtype=np.int64)
    span_splits = (seq_len + split_keys - 1) // split_keys - lo_req // split_keys
    can_split = (m_tiles <= MAX_SPLIT_TILES) & (span_splits > 1)
    n_splits = np.where(can_split, span_splits, 1)
    if fixed_splits:
        if (n_splits > fixed_splits).any() or (m_tiles != 1).any():
            raise ValueError("a fixed-size work list needs one row tile per request and "
                             "no more splits than its capacity")
        per_req = np.full(R, fixed_splits, dtype=np.int64)
    else:
        per_req = m_tiles * n_splits
    total = int(per_req.sum())
    req = np.repeat(np.arange(R, dtype=np.int64), per_req)
    first = np.cumsum(per_req) - per_req
    local = np.arange(total, dtype=np.int64) - np.repeat(first, per_req)
    ns = n_splits[req]
    work = np.empty((total, 4), dtype=np.int32)
    if fixed_splits:
        idle = local >= ns
        work[:, 0] = np.where(idle, -1, req)
        work[:, 1] = 0
        work[:, 2] = np.where(idle, 0, local)
    else:
        work[:, 0] = req
        work[:, 1] = local // ns
        work[:, 2] = local % ns
    work[:, 3] = ns
    if not fixed_splits and total > 1 and (m_tiles > 1).any():
        # prompt portions: the tiles with the most keys first, so that the last blocks of the
        # launch are the short ones (the order of the list has no other meaning)
        mt = work[:, 1].astype(np.int64)
        qn, p0 = q_len[req], pos0[req]
        row_hi = np.minimum(qn - 1, ((mt + 1) * tile_rows - 1) // group_size)
        hi = p0 + row_hi + 1
        lo = np.maximum(0, p0 + (mt * tile_rows) // group_size - window + 1) if window else 0
        cost = np.where(ns > 1, np.minimum(split_keys, hi - lo), hi - lo)
        work = work[np.argsort(-cost, kind="stable")]
    T = int(q_len.sum())
    tok_split_row = np.full(T, -1, dtype=np.int32)
    is_split = (n_splits > 1) | force_split
    split_req = np.nonzero(is_split)[0]
    if len(split_req):
        rows_per = q_len[split_req]
        n_rows = int(rows_per.sum())
        sfirst = np.cumsum(rows_per) - rows_per
        rreq = np.repeat(split_req, rows_per)
        off = np.arange(n_rows, dtype=np.int64) - np.repeat(sfirst, rows_per)
        split_tokens = (q_start[rreq] + off).astype(np.int32)
        split_counts = n_splits[rreq].astype(np.int32)
        tok_split_row[split_tokens] = np.arange(n_rows, dtype=np.int32)
    else:
        split_tokens = np.zeros(0, dtype=np.int32)
        split_counts = np.zeros(0, dtype=np.int32)
    max_splits = int(fixed_splits or (n_splits.max() if R else 1))
    return work, tok_split_row, split_tokens, split_counts, max_splits


def work_kinds(work: np.ndarray, q_len: np.ndarray, group_size: int, tile_rows: int) -> int:
    """Which instances of the tensor-core attention kernel have work: bit 0 for row tiles of
    at most 16 packed rows (decoded tokens, tails), bit 1 for larger ones; and how many of the
    small ones there are."""
    live = work[:, 0] >= 0
    if not live.any():
        return 0, 0
    req = work[live, 0].astype(np.int64)
    rows = np.minimum(tile_rows, q_len[req].astype(np.int64) * group_size - work[live, 1].astype(np.int64) * tile_rows)
    small = rows <= 16
    return (1 if small.any() else 0) | (2 if (~small).any() else 0), int(small.sum())


class _Packer:
    """Collects int32 arrays into one buffer; hands out views after a single copy."""

    def __init__(self):
        self.parts: List[np.ndarray] = []
        self.offsets: List[Tuple[int, Tuple[int, ...]]] = []
        self.total = 0

    def add(self, a: np.ndarray) -> int:
        a = np.ascontiguousarray(a, dtype=np.int32)
        idx = len(self.parts)
        self.parts.append(a)
        self.offsets.append((self.total, a.shape))
        self.total += (a.size + 3) // 4 * 4      # keep every array 16-byte aligned
        return idx

    def upload(self, device, pinned: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None):
        n = max(self.total, 4)
        if pinned is None or pinned.numel() < n:
            pinned = torch.empty(n, dtype=torch.int32, pin_memory=torch.cuda.is_available())
        host = pinned.numpy()
        for a, (o, _) in zip(self.parts, self.offsets):
            host[o:o + a.size] = a.reshape(-1)
        if out is None or out.numel() < n:
            out = torch.empty(n, dtype=torch.int32, device=device)
        out[:n].copy_(pinned[:n], non_blocking=True)
        self.device_buffer = out
        self.pinned = pinned
        return out

    def view(self, idx: int) -> torch.Tensor:
        o, shape = self.offsets[idx]
        n = int(np.prod(shape)) if len(shape) else 1
        return self.device_buffer[o:o + n].view(shape)


class StepContext:
    """Everything the parts read about the step besides their input rows."""
    captured = False              # True for the fixed-layout context of a captured decode step

    def __init__(self, manager: CacheManager, entries: Sequence[StepEntry], device, work_keys,
                 vocab_size: Optional[int] = None, min_bt_stride: int = 1):
        self.manager = manager
        self.page_tokens = manager.page_tokens
        self.device = device
        P = self.page_tokens
        R = len(entries)
        if R == 0:
            raise ValueError("a step needs at least one entry")
        self.split_keys = choose_split_keys(R)
        q_len = np.array([len(e.tokens) for e in entries], dtype=np.int64)
        if (q_len <= 0).any():
            raise ValueError("every entry of a step brings at least one token")
        ctx_before = np.array([manager.context_len(e.handle) for e in entries], dtype=np.int64)
        for e, n, c in zip(entries, q_len, ctx_before):
            if manager.reserved_len(e.handle) < c + n:
                raise ValueError("a step's tokens must be backed by pages before it runs "
                                 "(reserve them with the cache manager)")
        seq_len = ctx_before + q_len
        q_start = np.cumsum(q_len) - q_len
        T = int(q_len.sum())
        self.num_tokens, self.num_requests = T, R
        self.q_len_host, self.seq_len_host, self.q_start_host = q_len, seq_len, q_start
        self.context_before_host = ctx_before
        self.state_slots_host = np.array([manager.state_slot(e.handle) for e in entries], dtype=np.int64)
        tokens = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries])
        if vocab_size is not None and ((tokens < 0) | (tokens >= vocab_size)).any():
            bad = tokens[(tokens < 0) | (tokens >= vocab_size)][0]
            raise ValueError(f"token id {int(bad)} is outside the vocabulary of {vocab_size}")
        req_of_tok = np.repeat(np.arange(R), q_len)
        offs = np.arange(T) - q_start[req_of_tok]
        positions = ctx_before[req_of_tok] + offs
        want_rows = []
        for r, e in enumerate(entries):
            for w in e.want:
                if not (0 <= int(w) < q_len[r]):
                    raise ValueError(f"wanted place {w} is outside the entry's {int(q_len[r])} tokens")
                want_rows.append(int(q_start[r]) + int(w))
        self.num_wanted = len(want_rows)
        # explicit position ids (all entries or none): [T, axes]
        given = [e.position_ids is not None for e in entries]
        pos_ids = None
        if any(given):
            if not all(given):
                raise ValueError("either every entry of a step brings position ids or none does")
            rows_ = [np.asarray(e.position_ids, dtype=np.int64).reshape(len(e.tokens), -1) for e in entries]
            if len({r_.shape[1] for r_ in rows_}) != 1:
                raise ValueError("the entries' position ids differ in their number of axes")
            pos_ids = np.concatenate(rows_, axis=0)

        pk = _Packer()
        i_tokens, i_pos = pk.add(tokens), pk.add(positions)
        i_pos_ids = pk.add(pos_ids) if pos_ids is not None else None
        i_qs, i_ql, i_sl = pk.add(q_start), pk.add(q_len), pk.add(seq_len)
        i_want = pk.add(np.array(want_rows, dtype=np.int64))
        i_state = pk.add(self.state_slots_host)
        i_groups = []
        for g in range(len(manager.groups)):
            tables = [manager.block_table(e.handle, g) for e in entries]
            stride = max(min_bt_stride, max(len(t) for t in tables))
            bt = np.full((R, stride), -1, dtype=np.int32)
            for r, t in enumerate(tables):
                bt[r, :len(t)] = t
            blk = positions // P
            page = bt[req_of_tok, blk]
            if (page < 0).any():
                raise ValueError("a token of this step lies in a page that is not held")
            slots = page.astype(np.int64) * P + positions % P
            i_groups.append((pk.add(bt), stride, pk.add(slots)))
        i_work = {}
        self._work_host = {}
        for key in work_keys:
            group, gsize, tile_rows, window = key
            work, tsr, st, sc, max_splits = attention_work_arrays(q_len, seq_len, q_start, gsize,
                                                                  tile_rows, window, split_keys=self.split_keys)
            i_work[key] = (pk.add(work), len(work), pk.add(tsr), pk.add(st), pk.add(sc), len(st),
                           max_splits, work_kinds(work, q_len, gsize, tile_rows))
        pk.upload(device)
        self._packer = pk
        self.token_ids = pk.view(i_tokens)
        self.positions = pk.view(i_pos)
        # what a position encoding is given: the explicit ids ([T] for one axis, [T, axes] for
        # several), or the places in the sequence
        self.position_ids = self.positions
        if i_pos_ids is not None:
            ids = pk.view(i_pos_ids)
            self.position_ids = ids.reshape(-1) if ids.shape[1] == 1 else ids
        self.q_start, self.q_len, self.seq_len = pk.view(i_qs), pk.view(i_ql), pk.view(i_sl)
        self.want_rows = pk.view(i_want)
        self.state_slots = pk.view(i_state)
        self._groups = [GroupArrays(pk.view(ib), stride, pk.view(isl)) for ib, stride, isl in i_groups]
        self._work: Dict[tuple, AttentionWork] = {}
        for key, (iw, nw, itsr, ist, isc, ns, max_splits, (kinds, small_items)) in i_work.items():
            g = self._groups[key[0]]
            self._work[key] = AttentionWork(
                q_start=self.q_start, q_len=self.q_len, seq_len=self.seq_len,
                block_table=g.block_table, bt_stride=g.bt_stride, work=pk.view(iw), num_work=nw,
                tok_split_row=pk.view(itsr), split_tokens=pk.view(ist) if ns else None,
                split_counts=pk.view(isc) if ns else None, num_split_rows=ns, max_splits=max_splits,
                split_keys=self.split_keys, tile_rows=key[2], kinds=kinds, small_items=small_items,
                decode_rows=R if int(q_len.max(initial=0)) == 1 and int(q_len.min(initial=1)) == 1 else 0,
                longest_keys=int(seq_len.max(initial=0)))

    def group(self, g: int) -> GroupArrays:
        return self._groups[g]

    def attention_work(self, group: int, group_size: int, tile_rows: int, window, num_heads: int,
                       head_dim: int) -> AttentionWork:
        w = self._work[(group, group_size, tile_rows, window)]
        few = w.small_items * (num_heads // group_size) <= ops.decode_block_max_items(self.device)
        w.kinds = (w.kinds & ~4) | (4 if few else 0)
        if w.num_split_rows and (w.part_o is None or w.part_o.shape[1] != num_heads
                                 or w.part_o.shape[3] != head_dim):
            w.part_o = torch.empty((w.num_split_rows, num_heads, w.max_splits, head_dim),
                                   dtype=torch.float32, device=self.device)
            w.part_ml = torch.empty((w.num_split_rows, num_heads, w.max_splits, 2),
                                    dtype=torch.float32, device=self.device)
        return w
