"""Which matrix-product kernel a projection of a step goes to: decided from the step's rows, the
projection and the size of the matrix alone (no GPU needed to check the rule)."""
import torch

from paged_batch_engine_b200.csrc import ops


def _bf16(rows, cols):
    return torch.empty((rows, cols), dtype=torch.bfloat16, device="meta")


def test_stream_mask_by_rows():
    assert ops.stream_mask(1) == ops.STREAM_MASK_FEW and ops.stream_mask(ops.SKINNY_MAX_ROWS) == ops.STREAM_MASK_FEW
    assert ops.stream_mask(ops.SKINNY_MAX_ROWS + 1) == ops.STREAM_MASK
    assert ops.stream_mask(ops.STREAM_MID_ROWS) == ops.STREAM_MASK
    assert ops.stream_mask(ops.STREAM_MID_ROWS + 1) == ops.STREAM_MASK_MANY
    assert ops.stream_mask(ops.STREAM_MAX_ROWS) == ops.STREAM_MASK_MANY
    assert ops.stream_mask(ops.STREAM_MAX_ROWS + 1) == 0


def test_stream_applies_to_large_matrices_of_the_masked_projections_only(monkeypatch):
    monkeypatch.setattr(ops, "STREAM_MASK_FEW", 4)
    monkeypatch.setattr(ops, "STREAM_MASK", 12)
    monkeypatch.setattr(ops, "STREAM_MASK_MANY", 4)
    monkeypatch.setattr(ops, "STREAM_MIN_WEIGHT", 48 << 20)
    big_gate_up, big_down = _bf16(37888, 3584), _bf16(3584, 18944)
    small_gate_up = _bf16(17920, 1536)
    for rows in (1, 8, 16, 33, 64):
        assert ops.stream_applies(_bf16(rows, 3584), big_gate_up, 4)
        assert not ops.stream_applies(_bf16(rows, 1536), small_gate_up, 4)      # below the size gate
        assert not ops.stream_applies(_bf16(rows, 3584), _bf16(4608, 3584), 1)  # QKV is in no default mask
    assert ops.stream_applies(_bf16(12, 18944), big_down, 8)                    # down: 9 to 16 rows only
    assert not ops.stream_applies(_bf16(8, 18944), big_down, 8)
    assert not ops.stream_applies(_bf16(40, 18944), big_down, 8)
    assert not ops.stream_applies(_bf16(65, 3584), big_gate_up, 4)              # more rows than the kernel's range
    assert not ops.stream_applies(torch.empty((8, 3584), dtype=torch.float32, device="meta"), big_gate_up, 4)
    assert not ops.stream_applies(_bf16(8, 3580), _bf16(37888, 3580), 4)        # rows not on 16-byte boundaries
    assert ops.stream_wanted(big_gate_up.numel()) and not ops.stream_wanted(small_gate_up.numel())


def test_skinny_and_tc5_rules(monkeypatch):
    w = _bf16(4608, 3584)
    assert ops.skinny_applies(_bf16(ops.SKINNY_MAX_ROWS, 3584), w)
    assert not ops.skinny_applies(_bf16(ops.SKINNY_MAX_ROWS + 1, 3584), w)
    monkeypatch.setattr(ops, "TC5_MASK", 0)
    assert not ops.tc5_applies(_bf16(2048, 3584), w, 1)
    monkeypatch.setattr(ops, "TC5_MASK", 4)
    assert ops.tc5_applies(_bf16(2048, 3584), w, 4) and not ops.tc5_applies(_bf16(2048, 3584), w, 1)
    assert not ops.tc5_applies(_bf16(ops.TC5_MIN_ROWS - 1, 3584), w, 4)
