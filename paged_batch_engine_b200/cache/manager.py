"""Host-side bookkeeping of the paged key/value cache and of per-request state slots.

What it owns: which physical page of which layer group belongs to which request, each
request's block table per group, how many tokens of a request are reserved and how many
are computed, and which fixed-size state slot a request has.  It owns no device memory
(``storage.py`` does) and launches nothing, so all of it is tested without a GPU.

The bookkeeping itself is C++ (``csrc/host/cache_manager.cpp``, built with g++ at first
use and called through ctypes); this module is its Python face and adds nothing but
argument checking and error messages.

In the reference the same duties are spread over ``base::BlockAllocator`` (one pool per
layer, FIFO free queue, refcounts, generations: infMain/source/base/block_allocator.cpp:
205-230, 264-282), ``base::SequenceKVManager`` (per-request page tables, transactional
append with rollback: infMain/source/base/sequence_kv_manager.cpp:204-299) and
``base::KVCacheManager`` (request handles made of slot and generation, stale handles
rejected: infMain/source/base/kv_cache_manager.cpp:44-59, 167-236, 756-784).  Differences
by design: a page id is valid for every layer of its group (the reference allocates all
layer pools in lock-step and then uses layer 0's table for all of them,
infMain/source/serving/mixed_batch_builder.cpp:150,190); layers with different needs
(all keys, or a window of keys) form groups with pools of their own; a windowed group
gives pages back as soon as the window has passed them.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np

_SLOT_BITS = 20
_SLOT_MASK = (1 << _SLOT_BITS) - 1
NO_PAGE = -1

_ERR_STALE, _ERR_FREED_TWICE, _ERR_BAD_ARG, _ERR_CORRUPT = -1, -2, -3, -4


class CacheError(RuntimeError):
    """Misuse of the cache manager: a stale handle, a page freed twice, and the like."""


@dataclass(frozen=True)
class KVGroupSpec:
    """Layers whose paged tensors have the same geometry and the same lifetime.  The manager
    itself reads ``layers`` and ``window`` only; ``tensors`` (records with ``name``, ``heads``,
    ``width``) says what the storage holds per token; without it the group is a key and a
    value tensor of ``num_kv_heads`` x ``head_dim``."""
    layers: Tuple[int, ...]          # cache layer indices of the model's run order
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None     # None: every key is kept; W: only the last W keys are read
    tensors: Optional[Tuple[object, ...]] = None

    def __post_init__(self):
        if self.tensors is None:
            from ..parts.base import CacheTensor
            object.__setattr__(self, "tensors", (CacheTensor("k", self.num_kv_heads, self.head_dim),
                                                 CacheTensor("v", self.num_kv_heads, self.head_dim)))


_lib = None


def _host():
    global _lib
    if _lib is None:
        from ..csrc.build import load_host_library
        lib = load_host_library("cache_manager")
        i32, i64, vp = ctypes.c_int, ctypes.c_int64, ctypes.c_void_p
        pi32, pi64 = ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int64)
        sig = {
            "pbe_cm_new": (vp, [i32, pi32, i32, pi32, i32, i32]),
            "pbe_cm_delete": (None, [vp]),
            "pbe_cm_add_request": (i64, [vp]),
            "pbe_cm_is_live": (i32, [vp, i64]),
            "pbe_cm_num_live": (i32, [vp]),
            "pbe_cm_context_len": (i64, [vp, i64]),
            "pbe_cm_reserved_len": (i64, [vp, i64]),
            "pbe_cm_max_reserved_len": (i64, [vp, vp, ctypes.c_int]),
            "pbe_cm_num_free_pages": (i32, [vp, i32]),
            "pbe_cm_pool_num_pages": (i32, [vp, i32]),
            "pbe_cm_pool_allocations": (i64, [vp, i32]),
            "pbe_cm_page_generation": (i32, [vp, i32, i32]),
            "pbe_cm_page_refcount": (i32, [vp, i32, i32]),
            "pbe_cm_pages_needed": (i32, [vp, i64, i64, pi32]),
            "pbe_cm_max_appendable": (i64, [vp, i64]),
            "pbe_cm_reserve": (i32, [vp, i64, i64]),
            "pbe_cm_commit": (i32, [vp, i64, i64]),
            "pbe_cm_truncate": (i32, [vp, i64, i64]),
            "pbe_cm_free": (i32, [vp, i64]),
            "pbe_cm_block_table": (i32, [vp, i64, i32, vp, i32]),
            "pbe_cm_set_free_order": (i32, [vp, i32, vp, i32]),
            "pbe_cm_check": (i32, [vp, ctypes.c_char_p, i32]),
            "pbe_cm_decode_fill": (i32, [vp, i32, vp, vp, vp, vp, vp, vp, vp, i32]),
            "pbe_cm_reserve_many": (None, [vp, i32, vp, i64, vp]),
            "pbe_cm_commit_many": (i32, [vp, i32, vp, vp]),
            "pbe_cm_live_handles": (i32, [vp, vp, i32]),
            "pbe_cm_share_page": (i32, [vp, i32, i32]),
            "pbe_cm_unshare_page": (i32, [vp, i32, i32]),
            "pbe_cm_page_owner": (i64, [vp, i32, i32]),
            "pbe_decode_work_fill": (i32, [i32, i32, i32, vp, i32, i32, vp, vp, vp, vp, vp, vp, i32]),
        }
        for name, (res, args) in sig.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


class PagePoolView:
    """Read-only view of one group's page pool."""

    def __init__(self, manager: "CacheManager", group: int):
        self._m, self._g = manager, group

    @property
    def num_pages(self) -> int:
        return _host().pbe_cm_pool_num_pages(self._m._h, self._g)

    @property
    def num_free(self) -> int:
        return _host().pbe_cm_num_free_pages(self._m._h, self._g)

    @property
    def allocations(self) -> int:
        return _host().pbe_cm_pool_allocations(self._m._h, self._g)

    @property
    def generation(self) -> List[int]:
        lib = _host()
        return [lib.pbe_cm_page_generation(self._m._h, self._g, p) for p in range(self.num_pages)]

    def refcount(self, page: int) -> int:
        return _host().pbe_cm_page_refcount(self._m._h, self._g, page)


class CacheManager:
    """Pages, block tables and state slots of all live requests.

    ``add_request`` gives a handle (slot and generation packed in one integer);
    ``reserve(handle, n)`` backs the next ``n`` tokens with pages in every group or
    changes nothing; ``commit(handle, n)`` marks them computed and gives back pages that
    a window has passed; ``free(handle)`` gives everything back.
    """

    def __init__(self, groups: Sequence[KVGroupSpec], page_tokens: int, num_pages,
                 max_requests: int = 256, state_bytes: int = 0, lifo: bool = False):
        if page_tokens <= 0:
            raise CacheError(f"page_tokens must be positive, got {page_tokens}")
        if max_requests <= 0 or max_requests > _SLOT_MASK:
            raise CacheError(f"max_requests must be in 1..{_SLOT_MASK}, got {max_requests}")
        self.groups = tuple(groups)
        self.page_tokens = int(page_tokens)
        if isinstance(num_pages, int):
            num_pages = [num_pages] * len(self.groups)
        num_pages = [int(n) for n in num_pages]
        if len(num_pages) != len(self.groups):
            raise CacheError("num_pages needs one entry per group")
        if any(n <= 0 for n in num_pages):
            raise CacheError(f"a page pool needs at least one page, got {num_pages}")
        self.max_requests = int(max_requests)
        self.state_bytes = int(state_bytes)
        n = len(self.groups)
        windows = (ctypes.c_int * max(n, 1))(*[(-1 if g.window is None else int(g.window)) for g in self.groups])
        pages = (ctypes.c_int * max(n, 1))(*num_pages)
        self._h = _host().pbe_cm_new(n, windows, self.page_tokens, pages, self.max_requests, 1 if lifo else 0)
        if not self._h:
            raise CacheError("the cache manager could not be created with these sizes")
        self.pools = [PagePoolView(self, g) for g in range(n)]
        self._need = (ctypes.c_int * max(n, 1))()
        self.state_slot_assignments = 0

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and _lib is not None:
            _lib.pbe_cm_delete(h)

    # ------------------------------------------------------------------ errors
    def _raise(self, code: int, handle=None, what: str = ""):
        if code == _ERR_STALE:
            raise CacheError(f"stale or malformed request handle {handle!r}")
        if code == _ERR_FREED_TWICE:
            raise CacheError("a page was freed twice or lies outside its pool")
        if code == _ERR_BAD_ARG:
            raise CacheError(f"{what or 'bad argument'}")
        raise CacheError(f"cache manager failure ({code}) {what}")

    def _handle(self, handle) -> int:
        if not isinstance(handle, int) or isinstance(handle, bool) or handle < 0:
            raise CacheError(f"malformed request handle {handle!r}")
        return handle

    # ------------------------------------------------------------------ handles
    def is_live(self, handle) -> bool:
        return isinstance(handle, int) and handle >= 0 and bool(_host().pbe_cm_is_live(self._h, handle))

    @property
    def num_live_requests(self) -> int:
        return _host().pbe_cm_num_live(self._h)

    def add_request(self, user_id=None) -> Optional[int]:
        """A new request with no tokens; None when every request slot is taken."""
        h = _host().pbe_cm_add_request(self._h)
        if h < 0:
            return None
        self.state_slot_assignments += 1
        return int(h)

    def state_slot(self, handle: int) -> int:
        """Index of the request's fixed-size state (row of the state tensor)."""
        if not self.is_live(handle):
            self._raise(_ERR_STALE, handle)
        return handle & _SLOT_MASK

    # ------------------------------------------------------------------ sizes
    def context_len(self, handle: int) -> int:
        v = _host().pbe_cm_context_len(self._h, self._handle(handle))
        if v < 0:
            self._raise(int(v), handle)
        return int(v)

    def max_reserved_len(self, handles: Sequence[int]) -> int:
        """The longest reserved length (context plus tokens in flight) among the requests."""
        n = len(handles)
        arr = (ctypes.c_int64 * max(n, 1))(*[int(h) for h in handles])
        v = _host().pbe_cm_max_reserved_len(self._h, ctypes.addressof(arr), n)
        if v < 0:
            raise CacheError("a request handle of this step is stale or unknown")
        return int(v)

    def reserved_len(self, handle: int) -> int:
        v = _host().pbe_cm_reserved_len(self._h, self._handle(handle))
        if v < 0:
            self._raise(int(v), handle)
        return int(v)

    def num_free_pages(self, group: int = 0) -> int:
        return _host().pbe_cm_num_free_pages(self._h, group)

    def pages_needed(self, handle: int, n_tokens: int) -> List[int]:
        """New pages per group that ``reserve(handle, n_tokens)`` would take."""
        rc = _host().pbe_cm_pages_needed(self._h, self._handle(handle), int(n_tokens), self._need)
        if rc < 0:
            self._raise(rc, handle)
        return [self._need[g] for g in range(len(self.groups))]

    def can_reserve(self, handle: int, n_tokens: int) -> bool:
        need = self.pages_needed(handle, n_tokens)
        return all(n <= self.num_free_pages(g) for g, n in enumerate(need))

    def max_appendable_tokens(self, handle: int) -> int:
        """How many more tokens fit: room in the last page plus the free pages, the
        smallest over the groups (infMain/source/serving/scheduler.cpp:23-34)."""
        v = _host().pbe_cm_max_appendable(self._h, self._handle(handle))
        if v < 0:
            self._raise(int(v), handle)
        return int(v)

    def capacity_tokens(self) -> int:
        """Tokens one request could hold with every page of the scarcest group."""
        if not self.groups:
            return 1 << 30
        return min(p.num_pages for p in self.pools) * self.page_tokens

    # ------------------------------------------------------------------ pages
    def reserve(self, handle: int, n_tokens: int) -> bool:
        """Back tokens [reserved, reserved + n) with pages in every group, or change nothing."""
        if n_tokens < 0:
            raise CacheError(f"cannot reserve {n_tokens} tokens")
        rc = _host().pbe_cm_reserve(self._h, self._handle(handle), int(n_tokens))
        if rc < 0:
            self._raise(rc, handle)
        return rc == 1

    def reserve_many(self, handles: Sequence[int], n_tokens: int = 1) -> List[bool]:
        """``reserve`` for several requests in one call (the decode phase of a step)."""
        R = len(handles)
        hs = np.asarray(handles, dtype=np.int64)
        ok = np.empty(R, dtype=np.int32)
        _host().pbe_cm_reserve_many(self._h, R, hs.ctypes.data, int(n_tokens), ok.ctypes.data)
        if (ok < 0).any():
            bad = int(np.nonzero(ok < 0)[0][0])
            self._raise(int(ok[bad]), handles[bad])
        return [bool(v) for v in ok]

    def commit_many(self, handles: Sequence[int], n_tokens: Sequence[int]) -> None:
        """``commit`` for several requests in one call (after a step)."""
        hs = np.asarray(handles, dtype=np.int64)
        ns = np.asarray(n_tokens, dtype=np.int64)
        rc = _host().pbe_cm_commit_many(self._h, len(hs), hs.ctypes.data, ns.ctypes.data)
        if rc < 0:
            self._raise(rc, None, "a commit exceeds its reservation")

    def commit(self, handle: int, n_tokens: int) -> None:
        """Mark ``n_tokens`` more as computed and give back what a window has passed.

        A query at position p of a windowed group reads keys p-W+1..p, so once ``computed``
        tokens are written, the next query (position ``computed``) needs nothing below
        ``computed - W + 1``; pages that end at or before it go back to the pool and their
        block-table entries become NO_PAGE."""
        rc = _host().pbe_cm_commit(self._h, self._handle(handle), int(n_tokens))
        if rc < 0:
            self._raise(rc, handle, f"commit of {n_tokens} tokens exceeds the reservation")

    def truncate(self, handle: int, n_tokens: int) -> None:
        """Keep only the first ``n_tokens`` tokens (gives back tail pages).  Not allowed
        below what a window has already released."""
        rc = _host().pbe_cm_truncate(self._h, self._handle(handle), int(n_tokens))
        if rc < 0:
            self._raise(rc, handle, f"cannot truncate to {n_tokens} tokens")

    def free(self, handle: int) -> None:
        rc = _host().pbe_cm_free(self._h, self._handle(handle))
        if rc < 0:
            self._raise(rc, handle)

    # ------------------------------------------------------------------ views
    def block_table(self, handle: int, group: int = 0) -> List[int]:
        lib = _host()
        n = lib.pbe_cm_block_table(self._h, self._handle(handle), group, None, 0)
        if n < 0:
            self._raise(n, handle)
        out = np.empty(max(n, 1), dtype=np.int32)
        lib.pbe_cm_block_table(self._h, handle, group, out.ctypes.data, n)
        return out[:n].tolist()

    def slot_of_token(self, handle: int, group: int, position: int) -> int:
        """page * page_tokens + offset of a token (infMain/source/base/sequence_kv_manager.cpp:41-52)."""
        table = self.block_table(handle, group)
        page = table[position // self.page_tokens]
        if page == NO_PAGE:
            raise CacheError(f"position {position} lies in a page that was given back")
        return page * self.page_tokens + position % self.page_tokens

    def page_generation(self, group: int, page: int) -> int:
        return _host().pbe_cm_page_generation(self._h, group, page)

    def page_owner(self, group: int, page: int) -> Optional[int]:
        """The handle of the request the page was handed to; None for a free page."""
        v = int(_host().pbe_cm_page_owner(self._h, group, page))
        if v == _ERR_BAD_ARG:
            raise CacheError(f"page {page} lies outside the pool of group {group}")
        return None if v < 0 else v

    def share_page(self, group: int, page: int) -> None:
        """One more hold on a page that is held (its reference count goes up): it stays out of
        the free queue when its request gives it back, until ``unshare_page`` lets go as well.
        Nothing in this engine shares pages yet (no prefix cache); the directory keeps the
        count so that a page can be held more than once."""
        rc = _host().pbe_cm_share_page(self._h, group, page)
        if rc < 0:
            self._raise(rc, None, f"page {page} of group {group} is not held: it cannot be shared")

    def unshare_page(self, group: int, page: int) -> None:
        rc = _host().pbe_cm_unshare_page(self._h, group, page)
        if rc < 0:
            self._raise(rc, None, f"page {page} of group {group} has no further hold to let go of")

    def set_free_order(self, group: int, pages: Sequence[int]) -> None:
        """Test hook: the order in which the free pages of a group will be handed out."""
        arr = np.asarray(list(pages), dtype=np.int32)
        rc = _host().pbe_cm_set_free_order(self._h, group, arr.ctypes.data, len(arr))
        if rc < 0:
            self._raise(rc, None, "the order must list every free page exactly once")

    def decode_fill(self, handles: np.ndarray, ctx_before: np.ndarray, state_slots: np.ndarray,
                    block_tables: Sequence[np.ndarray], slots: Sequence[np.ndarray], known: np.ndarray,
                    refresh: bool) -> None:
        """One decode step's integers for ``handles`` (int64 [R]), written in place: context
        lengths and state slots (int64 [R]), block-table rows (int32 matrices, only entries
        beyond ``known`` unless ``refresh``) and cache slots (int32 [R]) per group."""
        n = len(self.groups)
        bt_ptrs = (ctypes.c_void_p * max(n, 1))(*[a.ctypes.data for a in block_tables])
        strides = (ctypes.c_int * max(n, 1))(*[a.strides[0] // 4 for a in block_tables])
        sl_ptrs = (ctypes.c_void_p * max(n, 1))(*[a.ctypes.data for a in slots])
        rc = _host().pbe_cm_decode_fill(self._h, len(handles), handles.ctypes.data, ctx_before.ctypes.data,
                                        state_slots.ctypes.data, ctypes.addressof(bt_ptrs),
                                        ctypes.addressof(strides), ctypes.addressof(sl_ptrs),
                                        known.ctypes.data, 1 if refresh else 0)
        if rc == _ERR_STALE:
            self._raise(rc, None)
        if rc < 0:
            raise ValueError("a token of this step lies in a page that is not held")

    # ------------------------------------------------------------------ self check
    def check_invariants(self) -> None:
        """No page lost, held twice or both held and free; counts agree."""
        buf = ctypes.create_string_buffer(512)
        if _host().pbe_cm_check(self._h, buf, 512) != 0:
            raise CacheError(buf.value.decode())

    def live_handles(self) -> List[int]:
        """Handles of all live requests."""
        lib = _host()
        out = np.empty(max(self.max_requests, 1), dtype=np.int64)
        n = lib.pbe_cm_live_handles(self._h, out.ctypes.data, len(out))
        return [int(h) for h in out[:n]]

    def reset(self) -> None:
        """Gives back everything every live request holds (a replay that starts over); handles
        handed out before go stale.  Page generations and allocation counts go on counting."""
        for h in self.live_handles():
            self.free(h)


def decode_work_fill(R: int, B: int, S: int, ctx_before: np.ndarray, window: Optional[int], split_keys: int,
                     work: np.ndarray, split_counts: np.ndarray, positions: Optional[np.ndarray],
                     seq_len: Optional[np.ndarray], tokens: Optional[np.ndarray],
                     token_values: Optional[np.ndarray], refresh: bool) -> int:
    """The attention work list of a captured decode step, written in place by the host library
    (see ``pbe_decode_work_fill``); returns the largest number of splits."""
    p = lambda a: a.ctypes.data if a is not None else None
    rc = _host().pbe_decode_work_fill(R, B, S, ctx_before.ctypes.data, int(window or 0), int(split_keys),
                                      p(work), p(split_counts), p(positions), p(seq_len), p(tokens),
                                      p(token_values), R if refresh else B)
    if rc < 0:
        raise ValueError("a request needs more key splits than this captured step holds")
    return rc
