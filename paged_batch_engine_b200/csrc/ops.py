"""Python faces of the CUDA entry points: each takes torch tensors on a CUDA device,
checks what the kernel assumes, and launches on the current stream.

There is no CPU path and no library stand-in for any of these: a tensor that is not on
a CUDA device is an error, and so is a failed build of the kernel library.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .build import load_library

c_void_p, c_int, c_float, c_ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else c_void_p(t.data_ptr())


def _stream():
    # the raw handle of the current stream, without building a torch.cuda.Stream object per launch
    return c_void_p(torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice()))


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("this engine runs on CUDA devices only: got a tensor on " + str(t.device))


def _need_contiguous(*tensors):
    for t in tensors:
        if t is not None and not t.is_contiguous():
            raise KernelError("kernel operands must be contiguous")


_launches = 0


def launch_count() -> int:
    """Kernel launches of this package issued from Python so far (a captured graph's
    launches count once, at capture)."""
    return _launches


def count_launches(n: int) -> None:
    """Launches made on this package's behalf by the host library."""
    global _launches
    _launches += int(n)


def _check(code: int, what: str):
    global _launches
    if code != 0:
        raise KernelError(f"{what}: CUDA error {code} at launch")
    _launches += 1




_fns = {}


def _fn(lib_name, fn_name, argtypes, defines=None):
    key = (lib_name, fn_name, tuple(sorted(defines.items())) if defines else None)
    fn = _fns.get(key)
    if fn is None:
        lib = load_library(lib_name, defines)
        fn = getattr(lib, fn_name)
        fn.argtypes = argtypes
        fn.restype = c_int
        _fns[key] = fn
    return fn


# ------------------------------------------------------------------ elementwise
def embedding(out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """out[t, :] = table[ids[t], :] as float32.  ids: int32 [T]."""
    _need_cuda(out, table, ids)
    _need_contiguous(out, table, ids)
    if out.dtype != torch.float32 or ids.dtype != torch.int32:
        raise KernelError("embedding writes float32 rows from int32 ids")
    T, d = out.shape
    if table.shape[1] != d or ids.numel() != T:
        raise KernelError("embedding: shapes do not agree")
    fn = _fn("elementwise", "pbe_embedding",
             [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(out), _ptr(table), _dtype_code(table), _ptr(ids), T, d, table.shape[0], _stream()),
           "embedding")
    return out


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], gain: torch.Tensor,
                out: torch.Tensor, eps: float, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """residual += delta (float32, in place) and out = rmsnorm(residual) * gain.

    With ``rows`` (int32 [n]) output row i is made from batch row rows[i] and the residual
    is not written."""
    _need_cuda(residual, delta, gain, out, rows)
    _need_contiguous(residual, delta, gain, out, rows)
    if residual.dtype != torch.float32 or gain.dtype != torch.float32:
        raise KernelError("add_rmsnorm: the residual stream and the gain are float32")
    d = residual.shape[-1]
    n = out.shape[0] if out.dim() == 2 else 1
    if gain.numel() != d or out.shape[-1] != d or (delta is not None and delta.shape != residual.shape):
        raise KernelError("add_rmsnorm: shapes do not agree")
    if rows is None and n != residual.shape[0]:
        raise KernelError("add_rmsnorm: output rows do not match the batch")
    if rows is not None and (rows.dtype != torch.int32 or rows.numel() != n):
        raise KernelError("add_rmsnorm: rows must be int32, one per output row")
    if d * 4 > 200 * 1024:
        raise KernelError(f"add_rmsnorm: a row of {d} floats does not fit in shared memory")
    fn = _fn("elementwise", "pbe_add_rmsnorm",
             [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_float,
              c_void_p])
    _check(fn(_ptr(residual), _ptr(delta), _dtype_code(delta) if delta is not None else F32,
              _ptr(gain), _ptr(out), _dtype_code(out), _ptr(rows), n, d, float(eps), _stream()),
           "add_rmsnorm")
    return out


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[r, c] = silu(gate_up[r, c]) * gate_up[r, inter + c]."""
    _need_cuda(gate_up, out)
    _need_contiguous(gate_up, out)
    rows, two_i = gate_up.shape
    if two_i % 2 or out.shape != (rows, two_i // 2) or out.dtype != gate_up.dtype:
        raise KernelError("silu_mul: shapes or dtypes do not agree")
    fn = _fn("elementwise", "pbe_silu_mul", [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(gate_up), _ptr(out), _dtype_code(out), rows, two_i // 2, _stream()), "silu_mul")
    return out


# ------------------------------------------------------------------ rope + cache write
def rope_kv_write(qkv: torch.Tensor, bias: Optional[torch.Tensor], q_out: torch.Tensor,
                  k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                  positions: torch.Tensor, slots: Optional[torch.Tensor],
                  inv_freq: Optional[torch.Tensor], num_heads: int, num_kv_heads: int,
                  head_dim: int, rotary_dim: int, page_tokens: int, interleaved: bool = False):
    """q_out = rope(q + b); cache[slot] = rope(k + b), v + b.  k_cache / v_cache are one
    layer's pages [page, kv_head, page_tokens, head_dim]; None: nothing is written."""
    _need_cuda(qkv, bias, q_out, k_cache, v_cache, positions, slots, inv_freq)
    _need_contiguous(qkv, bias, q_out, k_cache, v_cache, positions, slots, inv_freq)
    T = qkv.shape[0]
    width = (num_heads + 2 * num_kv_heads) * head_dim
    if qkv.shape[1] != width or q_out.shape != (T, num_heads * head_dim) or q_out.dtype != qkv.dtype:
        raise KernelError("rope_kv_write: shapes or dtypes do not agree")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != width):
        raise KernelError("rope_kv_write: bias must be float32 of the fused width")
    if positions.dtype != torch.int32 or positions.numel() != T:
        raise KernelError("rope_kv_write: positions must be int32 [T]")
    if k_cache is not None:
        if slots is None or slots.dtype != torch.int32 or slots.numel() != T:
            raise KernelError("rope_kv_write: slots must be int32 [T]")
        for c in (k_cache, v_cache):
            if c is None or c.dtype != qkv.dtype or tuple(c.shape[1:]) != (num_kv_heads, page_tokens, head_dim):
                raise KernelError("rope_kv_write: cache pages must be [page, kv_head, page_tokens, head_dim] "
                                  "in the activations' dtype")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.numel() != rotary_dim // 2):
        raise KernelError("rope_kv_write: inv_freq must be float32 [rotary_dim / 2]")
    fn = _fn("rope_kv", "pbe_rope_kv_write",
             [c_void_p] * 8 + [c_int] * 8 + [c_void_p])
    _check(fn(_ptr(qkv), _ptr(bias), _ptr(q_out), _ptr(k_cache), _ptr(v_cache), _ptr(positions),
              _ptr(slots), _ptr(inv_freq), T, num_heads, num_kv_heads, head_dim,
              rotary_dim if inv_freq is not None else 0, page_tokens, 1 if interleaved else 0,
              _dtype_code(qkv), _stream()), "rope_kv_write")
    return q_out


# ------------------------------------------------------------------ matrix products
def sgemm_nt(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor):
    """out = x @ w.T (+ bias) in true float32 arithmetic; w float32 [N, K]."""
    _need_cuda(x, w, bias, out)
    _need_contiguous(x, w, bias, out)
    M, K = x.shape
    N = w.shape[0]
    if w.dtype != torch.float32 or w.shape[1] != K or out.shape != (M, N):
        raise KernelError("sgemm_nt: shapes or dtypes do not agree")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError("sgemm_nt: bias must be float32 [N]")
    if x.dtype == torch.float32 and out.dtype != torch.float32:
        raise KernelError("sgemm_nt: float32 rows give float32 rows (bfloat16 rows give either)")
    need = _fn("sgemm", "pbe_sgemm_scratch_floats", [c_int, c_int, c_int, c_void_p])
    need.restype = c_ll
    n_tickets = c_int(0)
    floats = int(need(M, N, K, ctypes.byref(n_tickets)))
    scratch = tickets = None
    if floats > 0:
        # partial sums of the K slices, and the tickets by which the last block or warp of a group
        # of outputs learns that it is the one to add them up (zeroed once, left at zero by every call)
        scratch = torch.empty(floats, dtype=torch.float32, device=x.device)
        tickets = _sgemm_tickets.get(x.device)
        if tickets is None or tickets.numel() < n_tickets.value:
            tickets = _sgemm_tickets[x.device] = torch.zeros(max(8192, 2 * n_tickets.value), dtype=torch.int32,
                                                             device=x.device)
    fn = _fn("sgemm", "pbe_sgemm_nt",
             [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
              c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(x), _dtype_code(x), _ptr(w), _ptr(bias), _ptr(out), _dtype_code(out), M, N, K, K, N,
              _ptr(scratch), _ptr(tickets), _stream()), "sgemm_nt")
    return out


_sgemm_tickets = {}      # per device: zeroed int32 tickets shared by the float32 products of the stream


SKINNY_MAX_ROWS = int(os.environ.get('PBE_SKINNY_ROWS', '8'))      # batches of at most this many rows take the weight-streaming kernel (0: never); with 9 to
                         # 16 rows its two-tile instance loses to the library GEMM (4.39 against 3.48 ms a step)


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                out_dtype: Optional[torch.dtype] = None, swiglu: bool = False) -> torch.Tensor:
    """y = x w^T (+ b) for at most 16 rows, bfloat16 operands, weights streamed once.
    ``swiglu``: w is [gate; up] stacked and y = silu(x gate^T) * (x up^T), [M, N/2]."""
    _need_cuda(x, w, bias)
    _need_contiguous(x, w, bias)
    M, K = x.shape
    N = w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != K:
        raise KernelError("gemm_skinny takes bfloat16 x [M, K] and w [N, K]")
    if M > 16 or K % 8 != 0:
        raise KernelError(f"gemm_skinny takes at most 16 rows and K a multiple of 8 (got M={M}, K={K})")
    if swiglu and (N % 2 or bias is not None):
        raise KernelError("gemm_skinny: the SwiGLU epilogue needs an even N and no bias")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError("gemm_skinny: bias must be float32 [N]")
    out_dtype = out_dtype or torch.bfloat16
    out = torch.empty((M, N // 2 if swiglu else N), dtype=out_dtype, device=x.device)
    fn = _fn("gemm_skinny", "pbe_gemm_skinny",
             [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), _dtype_code(out), M, N, K, 1 if swiglu else 0,
              _stream()), "gemm_skinny")
    return out


_tc5_err = {}        # per device: the GEMM's flag
_tc5_attn_err = {}   # per device: the attention kernel's flag (element 0) and room for a debugging trace


TC5_PAIR = os.environ.get("PBE_TC5_PAIR", "0") == "1"


def gemm_tc5(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
             swiglu: bool = False, check: bool = False, pair: Optional[bool] = None) -> torch.Tensor:
    """y = x w^T for many rows on the tcgen05 tensor cores (TMA-fed, accumulator in tensor
    memory).  ``swiglu``: w is [gate; up] stacked and y = silu(x gate^T) * (x up^T), [M, N/2].
    ``pair``: two-SM tiles (a cluster of two blocks a 256 x 256 tile) from 256 rows on; None
    takes PBE_TC5_PAIR from the environment (off unless it is 1).
    ``check`` synchronises and raises if a bounded wait inside the kernel ran out."""
    _need_cuda(x, w)
    _need_contiguous(x, w)
    M, K = x.shape
    N = w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != K:
        raise KernelError("gemm_tc5 takes bfloat16 x [M, K] and w [N, K]")
    if K % 8 != 0:
        raise KernelError(f"gemm_tc5 needs K to be a multiple of 8 (rows on 16-byte boundaries), got {K}")
    out_dtype = out_dtype or torch.bfloat16
    if swiglu and (N % 2 or out_dtype != torch.bfloat16):
        raise KernelError("gemm_tc5: the SwiGLU epilogue needs an even N and bfloat16 output")
    out = torch.empty((M, N // 2 if swiglu else N), dtype=out_dtype, device=x.device)
    err = _tc5_err.get(x.device)
    if err is None:
        err = _tc5_err[x.device] = torch.zeros(1, dtype=torch.int32, device=x.device)
    fn = _fn("gemm_tc5", "pbe_gemm_tc5",
             [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    mode = (1 if swiglu else 0) | (2 if (TC5_PAIR if pair is None else pair) else 0)
    _check(fn(_ptr(x), _ptr(w), _ptr(out), _dtype_code(out), M, N, K, mode, _ptr(err), _stream()), "gemm_tc5")
    if check and int(err.item()) != 0:
        err.zero_()
        raise KernelError("gemm_tc5: a wait inside the kernel ran out; the result is invalid")
    return out


_stream_state = {}     # per device: (scratch floats, zeroed tickets) of the K-split products


def gemm_stream(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
                swiglu: bool = False, check: bool = False) -> torch.Tensor:
    """y = x w^T for up to 64 rows on the tcgen05 tensor cores with the weights as the streamed
    operand (TMA-fed ring, accumulator in tensor memory, K split over blocks where the matrix has
    few rows).  ``swiglu``: w is [gate; up] stacked and y = silu(x gate^T) * (x up^T), [M, N/2].
    ``check`` synchronises and raises if a bounded wait inside the kernel ran out."""
    _need_cuda(x, w)
    _need_contiguous(x, w)
    M, K = x.shape
    N = w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != K:
        raise KernelError("gemm_stream takes bfloat16 x [M, K] and w [N, K]")
    if M > STREAM_KERNEL_ROWS or K % 8 != 0:
        raise KernelError(f"gemm_stream takes at most {STREAM_KERNEL_ROWS} rows and K a multiple of 8 (got M={M}, K={K})")
    out_dtype = out_dtype or torch.bfloat16
    if swiglu and (N % 2 or out_dtype != torch.bfloat16):
        raise KernelError("gemm_stream: the SwiGLU epilogue needs an even N and bfloat16 output")
    out = torch.empty((M, N // 2 if swiglu else N), dtype=out_dtype, device=x.device)
    scratch, tickets, err = gemm_stream_buffers(x.device)
    fn = _fn("gemm_stream", "pbe_gemm_stream",
             [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(x), _ptr(w), _ptr(out), _dtype_code(out), M, N, K, 1 if swiglu else 0, _ptr(scratch), _ptr(tickets),
              _ptr(err), _stream()), "gemm_stream")
    if check and int(err.item()) != 0:
        err.zero_()
        raise KernelError("gemm_stream: a wait inside the kernel ran out; the result is invalid")
    return out


def gemm_stream_buffers(device):
    """(scratch, tickets, flag) of ``gemm_stream`` on this device, made on first use: partial tiles
    of at most one block a multiprocessor (128 weight rows x 64 batch rows of float32, twice that
    for gate and up), the tiles' tickets, zeroed once and left at zero by every launch, and the flag
    that a bounded wait sets."""
    device = torch.device(device)
    st = _stream_state.get(device)
    if st is None:
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        st = _stream_state[device] = (torch.empty(sms * 128 * 128, dtype=torch.float32, device=device),
                                      torch.zeros(1024, dtype=torch.int32, device=device))
    err = _tc5_err.get(device)
    if err is None:
        err = _tc5_err[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return st[0], st[1], err


# Which projections of a decode step go through gemm_stream, as bits (1 QKV, 2 output, 4 gate/up
# with SwiGLU, 8 down, 16 LM head and others): STREAM_MASK_FEW for steps of at most SKINNY_MAX_ROWS
# rows (the rest of such a step is gemm_skinny's), STREAM_MASK for steps of more rows up to
# STREAM_MID_ROWS and STREAM_MASK_MANY beyond that up to STREAM_MAX_ROWS (the rest is the
# library's).  Measured in the captured decode step of the 7B shape, ms a step: 1 / 2 / 4 / 8 rows
# with gate/up on it 2.91 / 2.93 / 2.98 / 3.12-3.14 against 2.95 / 2.99 / 3.05 / 3.19 on gemm_skinny
# (down on it as well: 3.14 at 8 rows, down alone 3.22); 16 rows 3.52 -> 3.37 with gate/up and
# down, 3.40 with all four; 24 / 32 / 48 / 64 rows with gate/up alone 3.67 / 3.76 / 4.18 / 4.52
# against 3.75 / 3.84 / 4.26 / 4.58 on the library GEMM and silu_mul (with down as well: level at 24
# and 32, 4.77 at 64).  So: gate/up everywhere up to 64 rows, down as well from 9 to 16.  The
# PBE_STREAM_FEW, PBE_STREAM and PBE_STREAM_MANY masks (0: never) and PBE_STREAM_ROWS /
# PBE_STREAM_MAX_ROWS override the choice.
STREAM_KERNEL_ROWS = 64
STREAM_MID_ROWS = int(os.environ.get("PBE_STREAM_ROWS", "16"))
STREAM_MAX_ROWS = min(STREAM_KERNEL_ROWS, int(os.environ.get("PBE_STREAM_MAX_ROWS", "64")))
STREAM_MASK_FEW = int(os.environ.get("PBE_STREAM_FEW", "4"))
STREAM_MASK = int(os.environ.get("PBE_STREAM", "12"))
STREAM_MASK_MANY = int(os.environ.get("PBE_STREAM_MANY", "4"))
# ... and only matrices of at least this many elements: below it (the 1.5B shape's 27.5 M and 13.8 M)
# the library's product is the shorter one (21.4 against 24.5 us, 19.5 against 20.5 us at 16 rows)
STREAM_MIN_WEIGHT = int(os.environ.get("PBE_STREAM_MIN_WEIGHT", str(48 << 20)))


def stream_mask(rows: int) -> int:
    if rows <= SKINNY_MAX_ROWS:
        return STREAM_MASK_FEW
    if rows <= STREAM_MID_ROWS:
        return STREAM_MASK
    return STREAM_MASK_MANY if rows <= STREAM_MAX_ROWS else 0


def stream_applies(x: torch.Tensor, w: torch.Tensor, bit: int) -> bool:
    return (stream_mask(x.shape[0]) & bit != 0 and x.dtype == torch.bfloat16
            and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and w.numel() >= STREAM_MIN_WEIGHT)


# Projections of many rows (prompt portions): which of them take gemm_tc5 instead of the vendor
# GEMM library, as bits (1 QKV, 2 output, 4 gate/up with the SwiGLU epilogue, 8 down, 16 others).
# PBE_GEMM in the environment: "tc5" all of them, "library" none, or the mask as a number.
def _tc5_mask() -> int:
    e = os.environ.get("PBE_GEMM", "").strip().lower()
    if e == "tc5":
        return 31
    if e == "library":
        return 0
    return int(e) if e.isdigit() else TC5_DEFAULT_MASK


TC5_DEFAULT_MASK = 0
TC5_MIN_ROWS = 128
TC5_MASK = _tc5_mask()


def tc5_applies(x: torch.Tensor, w: torch.Tensor, bit: int = 16) -> bool:
    return (TC5_MASK & bit != 0 and x.shape[0] >= TC5_MIN_ROWS and x.dtype == torch.bfloat16
            and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0)


def stream_wanted(largest_weight: int) -> bool:
    """True when a matrix of that many elements would go through gemm_stream at some step size."""
    return bool(STREAM_MASK or STREAM_MASK_FEW or STREAM_MASK_MANY) and largest_weight >= STREAM_MIN_WEIGHT


def gemm_libraries(dtype: torch.dtype, largest_weight: int = 0):
    """The matrix-product libraries a part of this dtype launches whose largest matrix has that
    many elements (for parallel builds)."""
    if dtype == torch.float32:
        return [("sgemm", None)]
    return [("gemm_skinny", None)] + ([("gemm_stream", None)] if stream_wanted(largest_weight) else []) + \
        ([("gemm_tc5", None)] if TC5_MASK else [])


def skinny_applies(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (0 < x.shape[0] <= SKINNY_MAX_ROWS and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and x.shape[1] % 8 == 0)


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None, kind: int = 16) -> torch.Tensor:
    """y = x w^T (+ b).  A float32 weight takes the true-float32 kernel of this package; a
    bfloat16 weight takes the package's weight-streaming kernels for few rows and otherwise the
    vendor GEMM library with float32 accumulation, as the reference does for every projection
    (matmul_kernel_batch.cu:39-208).  ``kind``: which projection this is, a bit of STREAM_MASK."""
    _need_cuda(x, w, bias)
    out_dtype = out_dtype or x.dtype
    if w.dtype == torch.float32:
        out = torch.empty((x.shape[0], w.shape[0]), dtype=out_dtype, device=x.device)
        return sgemm_nt(x, w, bias, out)
    if x.dtype != torch.bfloat16:
        raise KernelError("a bfloat16 weight takes bfloat16 activations")
    if bias is None and stream_applies(x, w, kind):
        return gemm_stream(x, w, out_dtype)
    if skinny_applies(x, w):
        return gemm_skinny(x, w, bias, out_dtype)
    if tc5_applies(x, w, kind) and bias is None:
        return gemm_tc5(x, w, out_dtype)
    if out_dtype == torch.float32:
        y = torch.mm(x, w.t(), out_dtype=torch.float32)
    else:
        y = torch.mm(x, w.t())
    if bias is not None:
        y += bias.to(y.dtype)
    return y


# ------------------------------------------------------------------ attention
class AttnParams(ctypes.Structure):
    _fields_ = [("q", c_void_p), ("k_cache", c_void_p), ("v_cache", c_void_p), ("out", c_void_p),
                ("part_o", c_void_p), ("part_ml", c_void_p), ("q_start", c_void_p),
                ("q_len", c_void_p), ("seq_len", c_void_p), ("block_table", c_void_p),
                ("work", c_void_p), ("tok_split_row", c_void_p),
                ("bt_stride", c_int), ("num_heads", c_int), ("num_kv_heads", c_int),
                ("page_tokens", c_int), ("window", c_int), ("split_keys", c_int),
                ("max_splits", c_int), ("tile_rows", c_int), ("scale", c_float), ("kinds", c_int),
                ("num_pages", c_int)]


class AttnMergeParams(ctypes.Structure):
    _fields_ = [("part_o", c_void_p), ("part_ml", c_void_p), ("out", c_void_p),
                ("split_tokens", c_void_p), ("split_counts", c_void_p),
                ("num_heads", c_int), ("head_dim", c_int), ("max_splits", c_int)]


SIMPLE_TILE_ROWS = 16   # packed rows per block of the plain attention kernel
SIMPLE_KEY_TILE = 32


def attention_kernel_config(head_dim: int, dtype: torch.dtype, kind: Optional[str] = None):
    """(kind, tile_rows, key_tile) of the attention kernel used for a head size and dtype."""
    if head_dim % 16 != 0 or head_dim <= 0 or head_dim > 256:
        raise KernelError(f"attention kernels take head sizes 16, 32, ..., 256; got {head_dim}")
    if kind is None and dtype == torch.bfloat16 and head_dim in (64, 128) and _attention_choice() != "mma" \
            and _tc5_available():
        kind = "tc5"
    kind = kind or ("mma" if dtype == torch.bfloat16 and _mma_available() else "simple")
    if kind == "simple":
        return "simple", SIMPLE_TILE_ROWS, SIMPLE_KEY_TILE
    if kind == "tc5":
        return "tc5", 128, 128
    return "mma", (128 if head_dim <= 128 else 64), MMA_KEY_TILE


MMA_KEY_TILE = 64


def _attention_choice() -> str:
    """Prompt portions of bfloat16 models with head size 64 or 128 run on the tcgen05
    attention kernel; PBE_ATTN=mma keeps them on the mma.sync kernel."""
    return os.environ.get("PBE_ATTN", "").strip().lower()


def _tc5_available() -> bool:
    from .build import KERNEL_DIR
    return os.path.isfile(os.path.join(KERNEL_DIR, "attention_tc5.cu"))


def _mma_available() -> bool:
    from .build import KERNEL_DIR
    return os.path.isfile(os.path.join(KERNEL_DIR, "attention_mma.cu"))


def paged_attention(q, k_cache, v_cache, out, meta, num_heads, num_kv_heads, head_dim, scale, window,
                    page_tokens, kind="simple"):
    """Causal attention of every row of the batch over the paged cache.

    ``meta`` carries the step's device arrays for this (group, head grouping, tile size,
    window): q_start, q_len, seq_len, block_table [R, stride], work [n, 4], tok_split_row,
    split_tokens, split_counts, max_splits, split_keys, part_o, part_ml."""
    _need_cuda(q, k_cache, v_cache, out)
    _need_contiguous(q, k_cache, v_cache, out)
    if q.dtype != k_cache.dtype or q.dtype != out.dtype:
        raise KernelError("attention: q, cache and output must share one dtype")
    if kind == "mma" and q.dtype != torch.bfloat16:
        raise KernelError("the tensor-core attention kernel takes bfloat16")
    lib = "attention_simple" if kind == "simple" else "attention_mma"
    defines = {"PBE_HEAD_DIM": int(head_dim)}
    tc5 = kind == "tc5"
    if tc5:
        if q.dtype != torch.bfloat16 or head_dim not in (64, 128):
            raise KernelError("the tcgen05 attention kernel takes bfloat16 and head sizes 64 and 128")
        # its page loads need pages of 8 tokens or more that divide the key tile of 64 or are a
        # multiple of it; with other page sizes the mma.sync kernel (same work list, same tile
        # rows) does the tiles
        tc5 = tc5_attention_applies(head_dim, page_tokens)
        kind = "mma"
    p = AttnParams(
        q=q.data_ptr(), k_cache=k_cache.data_ptr(), v_cache=v_cache.data_ptr(), out=out.data_ptr(),
        part_o=meta.part_o.data_ptr() if meta.part_o is not None else None,
        part_ml=meta.part_ml.data_ptr() if meta.part_ml is not None else None,
        q_start=meta.q_start.data_ptr(), q_len=meta.q_len.data_ptr(), seq_len=meta.seq_len.data_ptr(),
        block_table=meta.block_table.data_ptr(), work=meta.work.data_ptr(),
        tok_split_row=meta.tok_split_row.data_ptr(), bt_stride=int(meta.bt_stride),
        num_heads=int(num_heads), num_kv_heads=int(num_kv_heads), page_tokens=int(page_tokens),
        window=int(window or 0), split_keys=int(meta.split_keys), max_splits=int(meta.max_splits),
        tile_rows=int(meta.tile_rows), scale=float(scale), kinds=int(getattr(meta, "kinds", 0)),
        num_pages=int(k_cache.shape[0]))
    if tc5:
        # prompt-portion tiles on the tcgen05 kernel; the decode instances below take the rest
        err = tc5_attention_error_buffer(q.device)
        tfn = _fn("attention_tc5", "pbe_attn_tc5", [ctypes.POINTER(AttnParams), c_int, c_int, c_void_p, c_void_p],
                  defines)
        if (p.kinds & 3) == 0 or (p.kinds & 2):
            _check(tfn(ctypes.byref(p), int(meta.num_work), int(k_cache.shape[0]), _ptr(err), _stream()),
                   "paged_attention (tcgen05)")
        p.kinds = (p.kinds | 8) if (p.kinds & 3) else (1 | 8)
    fn = _fn(lib, "pbe_attn_" + kind, [ctypes.POINTER(AttnParams), c_int, c_int, c_void_p], defines)
    if kind == "mma":
        _mma_flag_heads.add(int(head_dim))
    _check(fn(ctypes.byref(p), int(meta.num_work), _dtype_code(q), _stream()), "paged_attention")
    if meta.num_split_rows > 0:
        mp = AttnMergeParams(part_o=meta.part_o.data_ptr(), part_ml=meta.part_ml.data_ptr(),
                             out=out.data_ptr(), split_tokens=meta.split_tokens.data_ptr(),
                             split_counts=meta.split_counts.data_ptr(), num_heads=int(num_heads),
                             head_dim=int(head_dim), max_splits=int(meta.max_splits))
        mfn = _fn("attention_simple", "pbe_attn_merge",
                  [ctypes.POINTER(AttnMergeParams), c_int, c_int, c_void_p], defines)
        _check(mfn(ctypes.byref(mp), int(meta.num_split_rows), _dtype_code(out), _stream()),
               "attention merge")
    return out


# The block-cooperative instance of the decode attention kernel (four warps share each key tile)
# is the shortest path through one work item; it pays while all its blocks (work items x kv
# heads) are resident at once, three a multiprocessor.  Beyond that the persistent instance,
# in which every warp streams whole work items, is faster (measured crossover between 256 and
# 512 items on 148 multiprocessors).
DECODE_BLOCK_ITEMS_PER_SM = 3


_sm_counts = {}


def decode_block_max_items(device) -> int:
    sms = _sm_counts.get(device)
    if sms is None:
        try:
            sms = torch.cuda.get_device_properties(device).multi_processor_count
        except (RuntimeError, AssertionError):
            sms = 148
        _sm_counts[device] = sms
    return DECODE_BLOCK_ITEMS_PER_SM * sms


class AttnFusedParams(ctypes.Structure):
    _fields_ = [("qkv", c_void_p), ("bias", c_void_p), ("positions", c_void_p), ("slots", c_void_p),
                ("inv_freq", c_void_p), ("num_requests", c_int)]


FUSED_DECODE_MAX_KEYS_PER_BLOCK = 32768   # beyond that the other path takes the step


def fused_decode_splits(num_requests: int, num_kv_heads: int, longest_keys: int, device) -> int:
    """Blocks per (request, key/value head) of the fused decode attention kernel: the largest of
    8, 4, 2, 1 with which every block of the step is resident at once; 1 for steps too large for
    that (their blocks run in waves: batch 128 at 2,048 tokens 16,900 -> 20,600 tok/s against the
    separate kernels); 0 when a block would get more keys than the kernel is meant for."""
    cap = decode_block_max_items(device)
    for splits in (8, 4, 2, 1):
        blocks = num_requests * num_kv_heads * splits
        if blocks <= cap:
            per_block = (longest_keys + splits - 1) // splits
            if not 0 < per_block <= FUSED_DECODE_MAX_KEYS_PER_BLOCK:
                return 0
            # a few dozen blocks with thousands of keys each (one or two requests with very long
            # contexts) stream better as many small work items on the other path
            if per_block > 1536 and blocks <= 64:
                return 0
            return splits
    return 1 if 0 < longest_keys <= FUSED_DECODE_MAX_KEYS_PER_BLOCK else 0


def fused_decode_attention_applies(dtype: torch.dtype, head_dim: int, group_size: int) -> bool:
    return (dtype == torch.bfloat16 and head_dim % 16 == 0 and head_dim <= 256 and group_size <= 16
            and _mma_available() and os.environ.get("PBE_DECODE_FUSED", "1") != "0")


def attention_decode_fused(qkv, bias, k_cache, v_cache, out, meta, positions, slots, inv_freq, num_requests,
                           num_heads, num_kv_heads, head_dim, scale, window, page_tokens, splits=8):
    """A step of decoded tokens only (one row a request): bias and rotary position encoding of
    the new token's query, key and value, the cache write, attention over the pages and the
    merge of the key splits in ONE launch (clusters of 8 blocks, one per request and key/value
    head).  ``qkv``: the fused projection's output [T, (H + 2 KV) hd]; ``out``: [T, H hd];
    row r of both belongs to request r (a step of decoded tokens has its rows in that order)."""
    _need_cuda(qkv, bias, k_cache, v_cache, out, positions, slots, inv_freq)
    _need_contiguous(qkv, k_cache, v_cache, out)
    if qkv.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("the fused decode attention kernel takes bfloat16")
    p = AttnParams(
        q=None, k_cache=k_cache.data_ptr(), v_cache=v_cache.data_ptr(), out=out.data_ptr(),
        part_o=None, part_ml=None,
        q_start=meta.q_start.data_ptr(), q_len=meta.q_len.data_ptr(), seq_len=meta.seq_len.data_ptr(),
        block_table=meta.block_table.data_ptr(), work=None, tok_split_row=None, bt_stride=int(meta.bt_stride),
        num_heads=int(num_heads), num_kv_heads=int(num_kv_heads), page_tokens=int(page_tokens),
        window=int(window or 0), split_keys=int(meta.split_keys), max_splits=int(splits),
        tile_rows=int(meta.tile_rows), scale=float(scale), kinds=1, num_pages=int(k_cache.shape[0]))
    f = AttnFusedParams(qkv=qkv.data_ptr(), bias=bias.data_ptr() if bias is not None else None,
                        positions=positions.data_ptr(), slots=slots.data_ptr(), inv_freq=inv_freq.data_ptr(),
                        num_requests=int(num_requests))
    fn = _fn("attention_mma", "pbe_attn_decode_fused",
             [ctypes.POINTER(AttnParams), ctypes.POINTER(AttnFusedParams), c_int, c_int, c_void_p],
             {"PBE_HEAD_DIM": int(head_dim)})
    _mma_flag_heads.add(int(head_dim))
    _check(fn(ctypes.byref(p), ctypes.byref(f), _dtype_code(qkv), int(splits), _stream()), "attention_decode_fused")
    return out


def tc5_attention_error_buffer(device) -> torch.Tensor:
    """Element 0: set by the tcgen05 attention kernel when a bounded wait ran out."""
    err = _tc5_attn_err.get(device)
    if err is None:
        err = _tc5_attn_err[device] = torch.zeros(1024, dtype=torch.int32, device=device)
    return err


def tc5_attention_applies(head_dim: int, page_tokens: int) -> bool:
    return head_dim in (64, 128) and page_tokens >= 8 and page_tokens % 8 == 0 and \
        (64 % page_tokens == 0 or page_tokens % 64 == 0)


def tc5_error_flag(device) -> int:
    """1 if a bounded wait inside a tcgen05 kernel ran out since the last call (then reset)."""
    err = _tc5_attn_err.get(torch.device(device))
    if err is None:
        return 0
    v = int(err[0].item())
    if v:
        err[:1].zero_()
    return v


def attention_mma_wait_flag(head_dim: int) -> int:
    """1 once a bounded wait for a key tile ran out inside the mma.sync attention kernels of this
    head size (never in a correct run; the launch's results are not valid then)."""
    fn = _fn("attention_mma", "pbe_attn_mma_wait_gave_up", [], {"PBE_HEAD_DIM": int(head_dim)})
    return int(fn())


# ------------------------------------------------------------------ the kernels' status word
_STATUS_NAMES = {}      # device -> names of the flags, in bit order
_status_state = {}      # device -> (addresses on the device, number of flags, key of the sources)
_mma_flag_heads = set() # head sizes whose mma.sync attention library this process has launched


def _status_sources(device):
    """(name, device address) of every flag a bounded wait of this package's kernels can set
    on ``device``, in a fixed order."""
    device = torch.device(device)
    out = []
    err = _tc5_attn_err.get(device)
    if err is not None:
        out.append(("tcgen05 attention", err.data_ptr()))
    err = _tc5_err.get(device)
    if err is not None:
        out.append(("tcgen05 GEMM", err.data_ptr()))
    for hd in sorted(_mma_flag_heads):
        fn = _fns.get(("attention_mma", "pbe_attn_mma_wait_flag_address", (("PBE_HEAD_DIM", hd),)))
        if fn is None:
            lib = load_library("attention_mma", {"PBE_HEAD_DIM": hd})
            fn = lib.pbe_attn_mma_wait_flag_address
            fn.argtypes, fn.restype = [], ctypes.c_ulonglong
            _fns[("attention_mma", "pbe_attn_mma_wait_flag_address", (("PBE_HEAD_DIM", hd),))] = fn
        with torch.cuda.device(device):
            addr = int(fn())
        if addr:
            out.append((f"mma.sync attention (head size {hd})", addr))
    return out[:32]


def collect_status(out: torch.Tensor) -> torch.Tensor:
    """Launches a kernel that writes into ``out`` (int32, one element, on the device) a word
    with bit i set when flag i of ``status_names(device)`` was set, and clears those flags.
    A flag is set by a kernel whose bounded wait ran out: the results of that launch are not
    valid.  Costs one launch of one thread; nothing waits."""
    _need_cuda(out)
    device = out.device
    # the flags' addresses are looked up again only when a new flag has come into being
    key = (device in _tc5_attn_err, device in _tc5_err, len(_mma_flag_heads))
    st = _status_state.get(device)
    if st is None or st[2] != key:
        import numpy as np
        src = _status_sources(device)
        addrs = torch.from_numpy(np.array([a for _, a in src] + [0], dtype=np.uint64).view(np.int64)).to(device)
        st = _status_state[device] = (addrs, len(src), key)
        _STATUS_NAMES[device] = [n for n, _ in src]
    fn = _fn("elementwise", "pbe_collect_status", [c_void_p, c_int, c_void_p, c_void_p])
    _check(fn(_ptr(st[0]), st[1], _ptr(out), _stream()), "collect_status")
    return out


def status_message(device, word: int) -> str:
    names = _STATUS_NAMES.get(torch.device(device), [])
    hit = [names[i] if i < len(names) else f"flag {i}" for i in range(32) if (int(word) >> i) & 1]
    return ("a bounded wait ran out inside: " + ", ".join(hit) +
            "; the results of that step are not valid (the flags have been cleared)")


def raise_on_kernel_status(device) -> None:
    """Synchronises, reads the kernels' flags and raises KernelError if one was set."""
    out = torch.zeros(1, dtype=torch.int32, device=device)
    word = int(collect_status(out).item())
    if word:
        raise KernelError(status_message(device, word))


def attention_libraries(head_dim: int, dtype: torch.dtype):
    """The (library, defines) pairs a model with this head size needs, for parallel builds."""
    jobs = [("attention_simple", {"PBE_HEAD_DIM": int(head_dim)})]
    if dtype == torch.bfloat16 and _mma_available():
        jobs.append(("attention_mma", {"PBE_HEAD_DIM": int(head_dim)}))
        if head_dim in (64, 128) and _attention_choice() != "mma" and _tc5_available():
            jobs.append(("attention_tc5", {"PBE_HEAD_DIM": int(head_dim)}))
    return jobs


# ------------------------------------------------------------------ sampling
def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Greedy token per row; ties go to the lowest id."""
    _need_cuda(logits, out)
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("argmax takes float32 logits with unit column stride")
    n, V = logits.shape
    if out is None:
        out = torch.empty(n, dtype=torch.int32, device=logits.device)
    fn = _fn("sampling", "pbe_argmax", [c_void_p, c_ll, c_int, c_int, c_void_p, c_void_p])
    _check(fn(_ptr(logits), logits.stride(0), n, V, _ptr(out), _stream()), "argmax")
    return out


def sample(logits, temperature, top_k, top_p, uniform, out=None) -> torch.Tensor:
    """One token per row with per-row temperature (float32), top_k (int32), top_p (float32)
    and uniform draw (float32)."""
    _need_cuda(logits, temperature, top_k, top_p, uniform, out)
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample takes float32 logits with unit column stride")
    n, V = logits.shape
    for t, dt in ((temperature, torch.float32), (top_k, torch.int32), (top_p, torch.float32),
                  (uniform, torch.float32)):
        if t.dtype != dt or t.numel() != n or not t.is_contiguous():
            raise KernelError("sample: per-row parameters must be contiguous, one per row")
    if out is None:
        out = torch.empty(n, dtype=torch.int32, device=logits.device)
    fn = _fn("sampling", "pbe_sample", [c_void_p, c_ll, c_int, c_int] + [c_void_p] * 6)
    _check(fn(_ptr(logits), logits.stride(0), n, V, _ptr(temperature), _ptr(top_k), _ptr(top_p),
              _ptr(uniform), _ptr(out), _stream()), "sample")
    return out


def seen_mark(seen: torch.Tensor, tokens: torch.Tensor, slots: Optional[torch.Tensor] = None, slot: int = -1) -> None:
    """seen[slots[i], tokens[i]] = 1 (``slots`` None: all in row ``slot``).  seen: uint8
    [slots, ld], tokens and slots int32 on the device; slots below 0 are skipped."""
    _need_cuda(seen, tokens, slots)
    if seen.dtype != torch.uint8 or tokens.dtype != torch.int32 or (slots is not None and slots.dtype != torch.int32):
        raise KernelError("seen_mark: a uint8 table, int32 tokens and slots")
    fn = _fn("sampling", "pbe_seen_mark", [c_void_p, c_ll, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p])
    _check(fn(_ptr(seen), seen.stride(0), seen.shape[1], _ptr(slots), int(slot), _ptr(tokens), tokens.numel(),
              _stream()), "seen_mark")


def penalty_seen(logits: torch.Tensor, seen: torch.Tensor, slots: torch.Tensor, penalties: torch.Tensor) -> torch.Tensor:
    """The repetition penalty from the table of seen tokens: row r of ``logits`` takes the
    tokens marked in seen[slots[r]] (slot below 0: the row is left alone)."""
    _need_cuda(logits, seen, slots, penalties)
    n, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1 or seen.dtype != torch.uint8 or \
            slots.dtype != torch.int32 or penalties.dtype != torch.float32 or slots.numel() != n or penalties.numel() != n:
        raise KernelError("penalty_seen: wrong dtypes or sizes")
    fn = _fn("sampling", "pbe_penalty_seen", [c_void_p, c_ll, c_int, c_int, c_void_p, c_ll, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(logits), logits.stride(0), n, V, _ptr(seen), seen.stride(0), _ptr(slots), _ptr(penalties),
              _stream()), "penalty_seen")
    return logits


def sample_set_mode(mode: int) -> None:
    """0 (default): the sampling kernel's binned selection with the radix descent behind it; 1: the
    radix descent only.  Both give the same token; the switch is for tests that compare them."""
    _fn("sampling", "pbe_sample_set_mode", [c_int])(int(mode))


def apply_penalty(logits, rows, tokens, penalties):
    """logits[rows[i], tokens[i]] is divided by penalties[i] when positive, multiplied
    otherwise; every (row, token) pair appears once."""
    _need_cuda(logits, rows, tokens, penalties)
    n = rows.numel()
    if logits.dtype != torch.float32 or rows.dtype != torch.int32 or tokens.dtype != torch.int32 \
            or penalties.dtype != torch.float32 or tokens.numel() != n or penalties.numel() != n:
        raise KernelError("apply_penalty: wrong dtypes or sizes")
    fn = _fn("sampling", "pbe_apply_penalty", [c_void_p, c_ll, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    _check(fn(_ptr(logits), logits.stride(0), logits.shape[1], _ptr(rows), _ptr(tokens),
              _ptr(penalties), n, _stream()), "apply_penalty")
    return logits
