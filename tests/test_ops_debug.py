"""The guard-band allocator used to catch out-of-bounds kernel writes (tool itself, on CPU tensors)."""
import pytest
import torch

from b200fw.ops.debug import GUARD_BYTES, CanaryError, canary_arena


def test_arena_routes_allocations_and_passes_when_untouched():
    with canary_arena(("cpu",)) as arena:
        a = torch.empty((3, 5), dtype=torch.bfloat16, device="cpu")
        b = torch.zeros(7, dtype=torch.float32, device="cpu")
        c = torch.empty_like(a)
        d = torch.zeros_like(b, dtype=torch.int64)
        e = torch.empty(4)                                  # no device given: not routed
        a.fill_(1.0)
        c.copy_(a)
        b += 2
        assert a.shape == (3, 5) and a.dtype == torch.bfloat16 and a.is_contiguous()
        assert a.data_ptr() % 256 == 0 or a.data_ptr() % 64 == 0      # payload keeps the allocator's alignment
        assert float(b.sum()) == 14.0 and int(d.sum()) == 0 and d.dtype == torch.int64
        assert torch.equal(a, c) and e.shape == (4,)
    assert len(arena.records) == 4 and arena.violations() == []
    assert torch.empty is not None and torch.empty(2, device="cpu").numel() == 2      # patches removed


def test_arena_reports_writes_on_either_side():
    with pytest.raises(CanaryError) as ei:
        with canary_arena(("cpu",)) as arena:
            t = torch.empty(10, dtype=torch.float32, device="cpu")          # 40 payload bytes, 216 slack bytes
            raw, nbytes, _ = arena.records[-1]
            assert nbytes == 40
            raw[GUARD_BYTES + nbytes] = 0                                   # one element past the end
            raw[GUARD_BYTES - 2] = 7                                        # two bytes before the start
            t.fill_(3.0)                                                    # legal writes do not matter
    msg = str(ei.value)
    assert "AFTER the tensor (first at offset 40" in msg and "BEFORE the tensor (nearest at offset -2)" in msg
    assert "test_ops_debug.py" in msg                                       # names the allocating call site
    # check=False leaves the verdict to the caller
    with canary_arena(("cpu",), check=False) as arena:
        torch.zeros(3, device="cpu")
        arena.records[-1][0][0] = 1
    assert len(arena.violations()) == 1
