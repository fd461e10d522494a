"""Dispatch of a projection to the tcgen05 tensor-core kernel."""
from __future__ import annotations


def apply(linear, x, out, n_rows: int, mode: int, stream: int) -> bool:
    """Run the tensor-core product if it takes these operands; False means the caller
    runs the plain kernel."""
    return False


def apply_gated(linear, x, act, n_rows: int, stream: int) -> bool:
    """act = silu(x . Wgate^T) * (x . Wup^T) in one kernel, for a row-concatenated
    [gate; up] weight.  False means the caller runs product and activation separately."""
    return False
