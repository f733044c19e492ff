"""Python face of ``pbe_attn_simple_noalloc``: split paged attention for callers that
cannot allocate device memory (a plugin in a host application that owns the device heap, a
loop that must stay clear of the allocator).  The partial results of split key ranges go
to a fixed 8 MiB array inside the kernel library instead of buffers the caller brings; see
``kernels/attention_noalloc.h`` for the contract (size limit, first call outside stream
capture, calls that overlap on the GPU race on the shared array).

This wrapper itself uses torch only to read pointers; the C entry point is what such
callers link against.
"""
from __future__ import annotations

import ctypes

import torch

from .build import load_library
from .ops import AttnMergeParams, AttnParams, KernelError, _dtype_code, _stream

def library(head_dim: int) -> ctypes.CDLL:
    return load_library("attention_noalloc", {"PBE_HEAD_DIM": int(head_dim)})


def scratch_floats(head_dim: int) -> int:
    """The size of the built-in scratch array in floats, asked of the library itself."""
    fn = library(head_dim).pbe_attn_noalloc_scratch_floats
    fn.argtypes, fn.restype = [], ctypes.c_longlong
    return int(fn())


def paged_attention_noalloc(q, k_cache, v_cache, out, meta, num_heads, num_kv_heads, head_dim, scale,
                            window, page_tokens) -> torch.Tensor:
    """Same result as ``ops.paged_attention(..., kind="simple")``; ``meta.part_o`` and
    ``meta.part_ml`` are not used.  Raises when the partial results would not fit the
    built-in scratch."""
    lib = library(head_dim)
    fn = lib.pbe_attn_simple_noalloc
    fn.argtypes = [ctypes.POINTER(AttnParams), ctypes.c_int, ctypes.POINTER(AttnMergeParams), ctypes.c_int,
                   ctypes.c_int, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    none = None
    a = AttnParams(
        q=q.data_ptr(), k_cache=k_cache.data_ptr(), v_cache=v_cache.data_ptr(), out=out.data_ptr(),
        part_o=none, part_ml=none, q_start=meta.q_start.data_ptr(), q_len=meta.q_len.data_ptr(),
        seq_len=meta.seq_len.data_ptr(), block_table=meta.block_table.data_ptr(),
        work=meta.work.data_ptr(), tok_split_row=meta.tok_split_row.data_ptr(),
        bt_stride=int(meta.bt_stride), num_heads=int(num_heads), num_kv_heads=int(num_kv_heads),
        page_tokens=int(page_tokens), window=int(window or 0), split_keys=int(meta.split_keys),
        max_splits=int(meta.max_splits), tile_rows=int(meta.tile_rows), scale=float(scale))
    m = AttnMergeParams(
        part_o=none, part_ml=none, out=out.data_ptr(),
        split_tokens=meta.split_tokens.data_ptr() if meta.num_split_rows else none,
        split_counts=meta.split_counts.data_ptr() if meta.num_split_rows else none,
        num_heads=int(num_heads), head_dim=int(head_dim), max_splits=int(meta.max_splits))
    rc = fn(ctypes.byref(a), int(meta.num_work), ctypes.byref(m), int(meta.num_split_rows), _dtype_code(q),
            _stream())
    if rc != 0:
        raise KernelError(f"pbe_attn_simple_noalloc: error {rc}")
    return out
