"""The decoder block enqueued by one call into the host library (``host/block_exec.cpp``).

``BlockDesc`` holds what a layer never changes (weights, sizes), ``StepDesc`` a step's buffers
and integers; ``run_block`` enqueues norm, QKV projection, position encoding and cache write,
attention, output projection, norm and feed-forward of one layer with the same kernels the
Python parts launch one by one.  It exists for steps that are not replayed from a captured
graph (prompt portions, mixed steps), where the interpreter's cost per launch, about 30 us,
adds up to milliseconds a step.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_void_p
from typing import Optional

import torch

from . import ops
from .build import load_host_library, load_library


class ExecFns(ctypes.Structure):
    _fields_ = [(n, c_void_p) for n in ("add_rmsnorm", "rope_kv_write", "gemm_skinny", "silu_mul", "attn_mma",
                                        "attn_tc5", "attn_merge", "attn_decode_fused", "cublas_gemm_ex",
                                        "gemm_stream")]


class BlockDesc(ctypes.Structure):
    _fields_ = [("w_qkv", c_void_p), ("b_qkv", c_void_p), ("w_o", c_void_p), ("w_gate_up", c_void_p),
                ("w_down", c_void_p), ("norm1", c_void_p), ("norm2", c_void_p), ("inv_freq", c_void_p),
                ("hidden", c_int), ("heads", c_int), ("kv_heads", c_int), ("head_dim", c_int), ("inter", c_int),
                ("eps1", c_float), ("eps2", c_float), ("scale", c_float), ("window", c_int), ("use_tc5", c_int)]


class StepDesc(ctypes.Structure):
    _fields_ = [("num_rows", c_int), ("residual", c_void_p), ("x", c_void_p), ("qkv", c_void_p), ("q", c_void_p),
                ("attn", c_void_p), ("gate_up", c_void_p), ("act", c_void_p), ("positions", c_void_p),
                ("slots", c_void_p), ("page_tokens", c_int), ("num_pages", c_int),
                ("attn_params", ops.AttnParams), ("num_work", c_int), ("num_split_rows", c_int),
                ("merge_params", ops.AttnMergeParams), ("fused_splits", c_int), ("decode_rows", c_int),
                ("tc5_pages_ok", c_int), ("tc5_err", c_void_p), ("cublas_handle", c_void_p),
                ("skinny_max_rows", c_int), ("stream_mid_rows", c_int), ("stream_max_rows", c_int), ("stream_mask_few", c_int), ("stream_mask", c_int),
                ("stream_mask_many", c_int),
                ("stream_min_weight", ctypes.c_longlong),
                ("stream_scratch", c_void_p), ("stream_tickets", c_void_p), ("stream_err", c_void_p)]


def enabled() -> bool:
    """PBE_EXEC=python keeps every launch in the interpreter; the opt-in tcgen05 GEMM for prompt
    portions has no place in the native block either."""
    return os.environ.get("PBE_EXEC", "native").strip().lower() != "python" and ops.TC5_MASK == 0


_host = None
_fns: dict = {}


def _addr(fn) -> int:
    return ctypes.cast(fn, c_void_p).value


def block_streams(block) -> bool:
    """True when one of the block's projections is large enough for gemm_stream."""
    m, f = block.mixer, block.ffn
    return ops.stream_wanted(max(t.numel() for t in (m.w_qkv, m.w_o, f.w_gate_up, f.w_down)))


def exec_fns(head_dim: int, use_tc5: bool, stream: bool = False) -> ExecFns:
    """The launchers' addresses for one head size (the attention libraries are built per head size);
    ``stream``: with gemm_stream's (a model of small matrices never launches it)."""
    key = (int(head_dim), bool(use_tc5), bool(stream))
    f = _fns.get(key)
    if f is None:
        defines = {"PBE_HEAD_DIM": int(head_dim)}
        ops._mma_flag_heads.add(int(head_dim))
        ew, rope, skinny = load_library("elementwise"), load_library("rope_kv"), load_library("gemm_skinny")
        mma, simple = load_library("attention_mma", defines), load_library("attention_simple", defines)
        cublas = ctypes.CDLL("libcublas.so.12")            # the one torch has loaded: its handle is used
        f = ExecFns(add_rmsnorm=_addr(ew.pbe_add_rmsnorm), rope_kv_write=_addr(rope.pbe_rope_kv_write),
                    gemm_skinny=_addr(skinny.pbe_gemm_skinny), silu_mul=_addr(ew.pbe_silu_mul),
                    attn_mma=_addr(mma.pbe_attn_mma),
                    attn_tc5=_addr(load_library("attention_tc5", defines).pbe_attn_tc5) if use_tc5 else None,
                    attn_merge=_addr(simple.pbe_attn_merge), attn_decode_fused=_addr(mma.pbe_attn_decode_fused),
                    cublas_gemm_ex=_addr(cublas.cublasGemmEx),
                    gemm_stream=_addr(load_library("gemm_stream").pbe_gemm_stream) if stream else None)
        _fns[key] = f
    return f


def _lib():
    global _host
    if _host is None:
        _host = load_host_library("block_exec")
        _host.pbe_exec_block.argtypes = [ctypes.POINTER(ExecFns), ctypes.POINTER(BlockDesc), ctypes.POINTER(StepDesc),
                                         c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]
        _host.pbe_exec_block.restype = c_int
        want = ctypes.sizeof(ExecFns) + ctypes.sizeof(BlockDesc) * 1000 + ctypes.sizeof(StepDesc)
        if _host.pbe_exec_abi() != want:
            raise ops.KernelError("the host library's structures and their ctypes mirrors differ in size")
    return _host


_STAGES = {1: "first norm", 2: "QKV projection", 3: "position encoding and cache write", 4: "attention",
           5: "merge of the key splits", 6: "output projection", 7: "second norm", 8: "gate/up projection",
           9: "activation", 10: "down projection"}


def run_block(block: BlockDesc, fns: ExecFns, step: StepDesc, delta_in: Optional[torch.Tensor],
              delta_out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor) -> None:
    rc = _lib().pbe_exec_block(ctypes.byref(fns), ctypes.byref(block), ctypes.byref(step),
                               delta_in.data_ptr() if delta_in is not None else None, delta_out.data_ptr(),
                               k_cache.data_ptr(), v_cache.data_ptr(), ops._stream())
    if rc < 0:
        stage, code = divmod(-rc, 1000000)
        raise ops.KernelError(f"native block: {_STAGES.get(stage, 'stage ' + str(stage))} failed with code {code}")
    ops.count_launches(rc)


def stage_profile(reset: bool = True) -> dict:
    """Host microseconds per call of each stage's launcher since the last reset."""
    ns = (ctypes.c_double * 16)()
    calls = (ctypes.c_longlong * 16)()
    _lib().pbe_exec_profile(ns, calls, 1 if reset else 0)
    return {_STAGES[i]: round(ns[i] / calls[i] / 1e3, 2) for i in _STAGES if calls[i]}


def block_desc(block) -> Optional[BlockDesc]:
    """The descriptor of a pre-norm block of RMSNorm, grouped-query attention with rotate-half
    rotary position encoding, and SwiGLU, all in bfloat16; None for anything else (those blocks
    run their parts from Python)."""
    from ..parts.attention import GQAttention
    from ..parts.mlp import SwiGLU
    from ..parts.norm import RMSNorm
    m, f, n1, n2 = getattr(block, "mixer", None), getattr(block, "ffn", None), getattr(block, "norm1", None), \
        getattr(block, "norm2", None)
    if not (type(m) is GQAttention and type(f) is SwiGLU and type(n1) is RMSNorm and type(n2) is RMSNorm):
        return None
    if m.dtype != torch.bfloat16 or m.o_bias or m.kernel_kind == "simple":
        return None
    tensors = [m.w_qkv, m.w_o, f.w_gate_up, f.w_down]
    if any(t is None or t.dtype != torch.bfloat16 or not t.is_contiguous() for t in tensors):
        return None
    if m.position.applies_itself:
        return None
    inv_freq, rotary_dim, interleaved = m.position.kernel_args()
    if inv_freq is None or rotary_dim != m.head_dim or interleaved:
        return None
    if not ops.fused_decode_attention_applies(m.dtype, m.head_dim, m.num_heads // m.num_kv_heads):
        return None
    return BlockDesc(w_qkv=m.w_qkv.data_ptr(), b_qkv=m.b_qkv.data_ptr() if m.b_qkv is not None else None,
                     w_o=m.w_o.data_ptr(), w_gate_up=f.w_gate_up.data_ptr(), w_down=f.w_down.data_ptr(),
                     norm1=n1.gain.data_ptr(), norm2=n2.gain.data_ptr(), inv_freq=inv_freq.data_ptr(),
                     hidden=m.hidden_size, heads=m.num_heads, kv_heads=m.num_kv_heads, head_dim=m.head_dim,
                     inter=f.intermediate_size, eps1=float(n1.eps), eps2=float(n2.eps), scale=float(m.scale),
                     window=int(m.window or 0), use_tc5=1 if m.kernel_kind == "tc5" else 0)


def _stream_fields(dev, block) -> dict:
    if not block_streams(block):
        return dict(stream_mid_rows=0, stream_max_rows=0, stream_mask_few=0, stream_mask=0, stream_mask_many=0,
                    stream_min_weight=0, stream_scratch=None, stream_tickets=None,
                    stream_err=None)
    scratch, tickets, err = ops.gemm_stream_buffers(dev)
    return dict(stream_mid_rows=int(ops.STREAM_MID_ROWS), stream_max_rows=int(ops.STREAM_MAX_ROWS),
                stream_mask_few=int(ops.STREAM_MASK_FEW), stream_mask=int(ops.STREAM_MASK),
                stream_mask_many=int(ops.STREAM_MASK_MANY),
                stream_min_weight=int(ops.STREAM_MIN_WEIGHT),
                stream_scratch=scratch.data_ptr(), stream_tickets=tickets.data_ptr(), stream_err=err.data_ptr())


def step_desc(block, ctx, cache, residual: torch.Tensor, buffers: dict) -> StepDesc:
    """A step's descriptor for the layers that share ``block``'s attention work list.  ``buffers``
    keeps the step's workspaces (allocated on first use, shared by all layers)."""
    m, f = block.mixer, block.ffn
    H, KV, hd = m.num_heads, m.num_kv_heads, m.head_dim
    T, dev, dt = residual.shape[0], residual.device, torch.bfloat16

    def buf(name, cols):
        t = buffers.get((name, cols))
        if t is None:
            t = buffers[(name, cols)] = torch.empty((T, cols), dtype=dt, device=dev)
        return t
    meta = ctx.attention_work(cache.group, H // KV, m.tile_rows, m.window, H, hd)
    group = ctx.group(cache.group)
    inv_freq, rotary_dim, interleaved = m.position.kernel_args()
    splits = m.fused_decode_splits(meta, cache, inv_freq, rotary_dim, interleaved)
    ap = ops.AttnParams(
        q=None, k_cache=None, v_cache=None, out=None,
        part_o=meta.part_o.data_ptr() if meta.part_o is not None else None,
        part_ml=meta.part_ml.data_ptr() if meta.part_ml is not None else None,
        q_start=meta.q_start.data_ptr(), q_len=meta.q_len.data_ptr(), seq_len=meta.seq_len.data_ptr(),
        block_table=meta.block_table.data_ptr(), work=meta.work.data_ptr(),
        tok_split_row=meta.tok_split_row.data_ptr(), bt_stride=int(meta.bt_stride), num_heads=H, num_kv_heads=KV,
        page_tokens=int(ctx.page_tokens), window=int(m.window or 0), split_keys=int(meta.split_keys),
        max_splits=int(meta.max_splits), tile_rows=int(meta.tile_rows), scale=float(m.scale),
        kinds=int(getattr(meta, "kinds", 0)))
    mp = ops.AttnMergeParams(part_o=ap.part_o, part_ml=ap.part_ml, out=None,
                             split_tokens=meta.split_tokens.data_ptr() if meta.num_split_rows else None,
                             split_counts=meta.split_counts.data_ptr() if meta.num_split_rows else None,
                             num_heads=H, head_dim=hd, max_splits=int(meta.max_splits))
    use_tc5 = m.kernel_kind == "tc5"
    err = ops.tc5_attention_error_buffer(dev) if use_tc5 else None
    # steps whose activation is the epilogue of the gate/up product need no [T, 2 inter] buffer
    fused_act = m.hidden_size % 8 == 0 and (T <= ops.SKINNY_MAX_ROWS or
                                            (ops.stream_mask(T) & 4 and
                                             2 * f.intermediate_size * m.hidden_size >= ops.STREAM_MIN_WEIGHT))
    big = not fused_act
    return StepDesc(
        num_rows=T, residual=residual.data_ptr(), x=buf("x", m.hidden_size).data_ptr(),
        qkv=buf("qkv", (H + 2 * KV) * hd).data_ptr(), q=buf("q", H * hd).data_ptr(),
        attn=buf("attn", H * hd).data_ptr(),
        gate_up=buf("gate_up", 2 * f.intermediate_size).data_ptr() if big else None,
        act=buf("act", f.intermediate_size).data_ptr(), positions=ctx.position_ids.data_ptr(),
        slots=group.slots.data_ptr(), page_tokens=int(ctx.page_tokens), num_pages=int(cache.k.shape[0]),
        attn_params=ap, num_work=int(meta.num_work), num_split_rows=int(meta.num_split_rows), merge_params=mp,
        fused_splits=int(splits), decode_rows=int(meta.decode_rows),
        tc5_pages_ok=1 if use_tc5 and ops.tc5_attention_applies(hd, ctx.page_tokens) else 0,
        tc5_err=err.data_ptr() if err is not None else None, cublas_handle=torch.cuda.current_blas_handle(),
        skinny_max_rows=int(ops.SKINNY_MAX_ROWS), **_stream_fields(dev, block))
