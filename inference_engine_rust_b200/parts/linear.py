"""A projection y = x . W^T with W stored [out, in] row-major, exactly as the weights
file has it (reference layout: src/ops/matmul.rs:1-3).  Not a registered part: mixers,
feed-forwards and the output head use it for their matrix products.

float32 runs use the plain fp32 kernel (every multiply-add in 32-bit).  bfloat16 runs use
the tcgen05 tensor-core kernel unless the runtime asks for plain kernels only.
"""
from __future__ import annotations

import torch

from typing import Optional, Union

from ..csrc import bindings as B
from .base import LazyInput, NormRequest, Runtime


def as_tensor(x: Union[torch.Tensor, LazyInput], n_rows: int) -> torch.Tensor:
    """`x` itself, or a lazy input computed into memory."""
    return x.materialize(n_rows) if isinstance(x, LazyInput) else x


class Linear:
    def __init__(self, weight: torch.Tensor, rt: Runtime):
        """`weight`: [out, in] on the device.  It is kept in the run's dtype: a matrix stored
        in 32-bit that feeds a bfloat16 product is rounded once, here."""
        if weight.dim() != 2:
            raise ValueError(f"a projection weight is 2-D, got shape {tuple(weight.shape)}")
        if weight.dtype != rt.dtype:
            weight = weight.to(rt.dtype)
        self.weight = weight.contiguous()
        self.out_features, self.in_features = self.weight.shape
        self.rt = rt
        self._fast = None

    def nbytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def apply(self, x: Union[torch.Tensor, LazyInput], out: torch.Tensor, n_rows: int, stream: int,
              add_residual: bool = False, ctx=None) -> None:
        """out[:n_rows] = x[:n_rows] . W^T, or out[:n_rows] += ... when `add_residual`
        (out is then the fp32 residual stream).  `x` may be a `LazyInput`: the kernel finishes it
        on the way if it can, else it is computed into memory first.  With `add_residual` and a
        step context whose `norm_ahead` is set, the kernel does the next norm's first half where
        it can and leaves the result in `ctx.rows_ahead`."""
        mode = B.GEMM_ADD_RESIDUAL if add_residual else B.GEMM_STORE
        if self.rt.fast:
            from . import fast_linear
            if fast_linear.apply(self, x, out, n_rows, mode, stream, ctx if add_residual else None):
                return
        B.gemm_plain(as_tensor(x, n_rows), self.weight, out, n_rows, mode, stream)
