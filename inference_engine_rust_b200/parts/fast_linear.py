"""Dispatch of a projection to the tcgen05 tensor-core kernel."""
from __future__ import annotations

import torch

from ..csrc import bindings as B


# The fused kernel puts 128 tokens on the MMA's M side and cannot split K: below this many
# tokens the separate product (split-K, thin token tile) + activation is faster.
GATED_MIN_ROWS = 128
# Up to this many tokens (decoding) the fused kernel has a second form: weight rows on the
# MMA's M side, 64 gate rows and their 64 up rows per tile.  It does not split K either and
# refuses when its tiles alone do not fill the device.
GATED_MAX_DECODE_ROWS = 64


def apply(linear, x, out, n_rows: int, mode: int, stream: int) -> bool:
    """Run the tensor-core product if it takes these operands (bf16, K and row strides
    multiples of 8, 16-byte aligned); False means nothing was launched and the caller runs the
    plain kernel."""
    if x.dtype != torch.bfloat16 or linear.weight.dtype != torch.bfloat16:
        return False
    return B.gemm_tc(x, linear.weight, out, n_rows, mode, linear.rt.err, stream)


def apply_gated(linear, x, act, n_rows: int, stream: int) -> bool:
    """act = silu(x . Wgate^T) * (x . Wup^T) in one kernel, for a row-concatenated
    [gate; up] weight.  False means the caller runs product and activation separately."""
    if x.dtype != torch.bfloat16 or linear.weight.dtype != torch.bfloat16 or act.dtype != torch.bfloat16:
        return False
    if n_rows < GATED_MIN_ROWS:
        # decoding: only the weight-major form, and only when 64-row tiles fill the device
        if n_rows > GATED_MAX_DECODE_ROWS or -(-(linear.weight.shape[0] // 2) // 64) < B.sm_count():
            return False
    return B.gemm_tc_gated(x, linear.weight, act, n_rows, linear.rt.err, stream)
