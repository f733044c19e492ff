"""The allocation-free attention entry point, called through its exported C symbol.

Some users of this library cannot call cudaMalloc: a plugin that lives inside a host
application which owns the device heap, or a serving loop that must never wait on the
allocator.  For them ``pbe_attn_simple_noalloc`` keeps the partial results of split key
ranges in a fixed array inside the library.  This test checks that it returns what the
regular entry points return (which take caller-allocated scratch), on two calls in a row
that share the built-in array, and that a request beyond the array's size is refused.

It is collected last so that a run which stops at the first failure has already run
every other test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(seed, reqs, dtype, H=6, KV=3, hd=48, P=8, window=None):
    from tests.test_gpu_kernels import AttnCase
    case = AttnCase(H, KV, hd, P, window, reqs, dtype, seed=seed, kind="simple")
    case.write_cache()
    regular = case.run()          # pbe_attn_simple + pbe_attn_merge with caller-allocated partials
    assert case.meta.num_split_rows > 0 and case.meta.max_splits > 1
    return case, regular


def _noalloc(case):
    from paged_batch_engine_b200.csrc.noalloc import paged_attention_noalloc
    qrows = torch.cat([q[c:c + n] for q, k, v, c, n, h in case.seqs]).reshape(-1, case.H * case.hd)
    out = torch.full_like(qrows, float("nan")).to(DEV)
    meta = case.meta
    saved = (meta.part_o, meta.part_ml)
    meta.part_o = meta.part_ml = None            # the caller brings no scratch
    try:
        paged_attention_noalloc(qrows.to(DEV).contiguous(), case.k_pages, case.v_pages, out, meta, case.H,
                                case.KV, case.hd, case.hd ** -0.5, case.window, case.P)
    finally:
        meta.part_o, meta.part_ml = saved
    torch.cuda.synchronize()
    return out.float().cpu().view(-1, case.H, case.hd)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_two_calls_in_a_row_match_the_regular_entry_points(dtype):
    """The kernels are the regular entry points' own, so the results are equal bit for bit;
    and the device's free memory does not move over the calls (a raw cudaMalloc inside the
    library, which torch's allocator would not see, would show here)."""
    first, want1 = _case(1, [(700, 1), (300, 2), (0, 40), (513, 1)], dtype)
    second, want2 = _case(2, [(1200, 1), (40, 1), (257, 3)], dtype, window=None)
    got1 = _noalloc(first)                        # the first call on the device: looks up the array
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    # inputs and outputs of the next calls come from torch's cache, not from the device heap
    got2 = _noalloc(second)                       # reuses the array the first call wrote
    got1_again = _noalloc(first)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    for got, want in ((got1, want1), (got2, want2), (got1_again, want1)):
        assert not torch.isnan(got).any()
        assert torch.equal(got, want)


def test_the_symbol_is_exported_and_refuses_what_does_not_fit():
    from paged_batch_engine_b200.csrc.noalloc import library, scratch_floats
    SCRATCH_FLOATS = scratch_floats(48)
    assert SCRATCH_FLOATS == 2 * 1024 * 1024             # the stated limit: 8 MiB
    from paged_batch_engine_b200.csrc.ops import AttnMergeParams, AttnParams
    lib = library(48)
    fn = lib.pbe_attn_simple_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.POINTER(AttnParams), ctypes.c_int, ctypes.POINTER(AttnMergeParams), ctypes.c_int,
                   ctypes.c_int, ctypes.c_void_p]
    a = AttnParams(num_heads=32, num_kv_heads=8, max_splits=64, tile_rows=16, split_keys=256, page_tokens=16)
    m = AttnMergeParams(num_heads=32, head_dim=48, max_splits=64)
    rows = SCRATCH_FLOATS // (32 * 64 * 50) + 1
    torch.cuda.synchronize()
    before = torch.cuda.mem_get_info()[0]
    assert fn(ctypes.byref(a), 1, ctypes.byref(m), rows, 0, None) == 1      # cudaErrorInvalidValue
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == before
