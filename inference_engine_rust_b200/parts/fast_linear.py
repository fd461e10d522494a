"""Dispatch of a projection to the tensor-core kernels."""
from __future__ import annotations

import os

import torch

from ..csrc import bindings as B
from .base import LazyInput
from .linear import as_tensor


# The fused kernel puts 128 tokens on the MMA's M side and cannot split K: below this many
# tokens the separate product (split-K, thin token tile) + activation is faster.
GATED_MIN_ROWS = 128
# Up to this many tokens (decoding) the fused kernel has a second form: weight rows on the
# MMA's M side, 64 gate rows and their 64 up rows per tile.  It does not split K either and
# refuses when its tiles alone do not fill the device.
GATED_MAX_DECODE_ROWS = 64


# One-token steps of up to this many tokens: a matrix whose 128-row tiles would not fill the device
# (the tcgen05 kernel would split k and add partial tiles through memory) goes to the kernel that
# gives every CTA 16 rows over all of k instead.
ROWS_KERNEL_MAX_TOKENS = int(os.environ.get("IERT_GEMM_ROWS_MAX", "16"))      # 0: never (for comparison)


def norm_ahead_enabled() -> bool:
    """IERT_NORM_AHEAD=0: every norm runs as a kernel of its own (for comparison)."""
    return os.environ.get("IERT_NORM_AHEAD", "1") != "0"


# One-token steps of up to this many tokens may split a norm around a kernel boundary (the weight-major
# tiles of the tcgen05 kernel end there).
NORM_AHEAD_MAX_TOKENS = 64


def apply(linear, x, out, n_rows: int, mode: int, stream: int, ctx=None) -> bool:
    """Run the tensor-core product if it takes these operands (bf16, K and row strides
    multiples of 8, 16-byte aligned); False means nothing was launched and the caller runs the
    plain kernel.  `x` may be the first half of a norm (`ScaledRows`); `ctx` (residual adds): its
    `norm_ahead`, if set, is honoured where the kernel can and the result left in `ctx.rows_ahead`."""
    from .norm import ScaledRows, honour
    if linear.weight.dtype != torch.bfloat16:
        return False
    err = linear.rt.err
    scaled = x if isinstance(x, ScaledRows) else None
    request = ctx.norm_ahead if ctx is not None and mode == B.GEMM_ADD_RESIDUAL else None
    thin = 2 * -(-linear.out_features // 128) <= 2 * B.sm_count()       # 128-row tiles alone would not fill the device
    if n_rows <= NORM_AHEAD_MAX_TOKENS and thin and (scaled is not None or request is not None or n_rows <= ROWS_KERNEL_MAX_TOKENS):
        xt = scaled.scaled if scaled is not None else as_tensor(x, n_rows)
        if xt.dtype == torch.bfloat16:
            ahead = finish = None
            if request is not None:
                parts = -(-linear.out_features // (16 if n_rows <= ROWS_KERNEL_MAX_TOKENS else 128))
                ahead, finish = honour(request, out, ctx, "linear", parts)
            scale = scaled.row_scale() if scaled is not None else None
            if n_rows <= ROWS_KERNEL_MAX_TOKENS:
                done = B.gemm_rows(xt, linear.weight, out, n_rows, mode, err, stream, scale=scale, ahead=ahead)
            else:
                done = (scale is not None or ahead is not None) and \
                    B.gemm_tc_scaled(xt, linear.weight, out, n_rows, mode, err, stream, scale=scale, ahead=ahead)
            if done:
                if finish is not None:
                    ctx.rows_ahead = finish()
                return True
    x = as_tensor(x, n_rows)
    if x.dtype != torch.bfloat16:
        return False
    return B.gemm_tc(x, linear.weight, out, n_rows, mode, err, stream)


def apply_gated(linear, x, act, n_rows: int, stream: int) -> bool:
    """act = silu(x . Wgate^T) * (x . Wup^T) in one kernel, for a row-concatenated
    [gate; up] weight.  False means the caller runs product and activation separately.  An `x`
    that is the first half of a norm (`ScaledRows`) is taken by the one-token form only."""
    from .norm import ScaledRows
    if linear.weight.dtype != torch.bfloat16 or act.dtype != torch.bfloat16:
        return False
    scaled = x if isinstance(x, ScaledRows) else None
    if scaled is None and isinstance(x, LazyInput):
        return False
    if scaled is None and x.dtype != torch.bfloat16:
        return False
    if n_rows < GATED_MIN_ROWS:
        # decoding: only the weight-major form, and only when 64-row tiles fill the device
        if n_rows > GATED_MAX_DECODE_ROWS or -(-(linear.weight.shape[0] // 2) // 64) < B.sm_count():
            return False
        if scaled is not None:
            return B.gemm_tc_gated_scaled(scaled.scaled, linear.weight, act, n_rows, scaled.row_scale(), linear.rt.err, stream)
    elif scaled is not None:
        return False
    return B.gemm_tc_gated(x, linear.weight, act, n_rows, linear.rt.err, stream)
