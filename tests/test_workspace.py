"""The per-step arena and the row counts that library products are issued with (CPU)."""
import torch

from poor_mans_mamba_b200.engine import Workspace
from poor_mans_mamba_b200.kernels.ops import padded_rows


def test_padded_rows_recur():
    """Row counts are rounded so that few distinct shapes reach the GEMM library: multiples of 64
    up to 1,024 rows, of 128 up to 4,096, of 256 beyond; steps of up to 64 tokens keep their count."""
    for n in (1, 8, 33, 64):
        assert padded_rows(n) == n
    assert padded_rows(65) == 128 and padded_rows(128) == 128 and padded_rows(1000) == 1024
    assert padded_rows(1025) == 1152 and padded_rows(4000) == 4096
    assert padded_rows(4097) == 4352 and padded_rows(8192) == 8192
    seen = {padded_rows(n) for n in range(65, 8193)}
    assert len(seen) <= 15 + 24 + 16 + 1
    assert all(padded_rows(n) >= n and padded_rows(n) - n < max(64, n // 8) for n in range(1, 9000, 7))


def test_arena_keeps_scratch_rows_behind_matrices():
    ws = Workspace(torch.device("cpu"), 1 << 22)
    a = ws.alloc((100, 24), torch.bfloat16)
    b = ws.alloc((3, 24), torch.bfloat16)
    c = ws.alloc((40, 8), torch.float32)       # up to 64 rows: no padding
    d = ws.alloc((2, 100, 24), torch.bfloat16)  # not a matrix: no padding
    e = ws.alloc((7,), torch.float32)
    assert getattr(a, "_scratch_rows", 0) == 128 and not hasattr(c, "_scratch_rows") and not hasattr(d, "_scratch_rows")
    assert b.data_ptr() - a.data_ptr() >= 128 * 24 * 2          # the rows behind a belong to nobody else
    assert d.data_ptr() - c.data_ptr() >= 40 * 8 * 4 and e.data_ptr() - d.data_ptr() >= 2 * 100 * 24 * 2
    # the same requests after a reset get the same tensors back (and the mark/release stack works)
    ws.reset()
    a2 = ws.alloc((100, 24), torch.bfloat16)
    assert a2.data_ptr() == a.data_ptr() and a2 is a
    mark = ws.mark()
    x = ws.alloc((70, 16), torch.float32)
    ws.release(mark)
    y = ws.alloc((70, 16), torch.float32)
    assert x.data_ptr() == y.data_ptr()
    # a frozen arena refuses to grow
    ws.freeze()
    try:
        ws.alloc((1 << 22,), torch.float32)
        raise AssertionError("a frozen arena grew")
    except RuntimeError:
        pass
