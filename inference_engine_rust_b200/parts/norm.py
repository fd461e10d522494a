"""RMSNorm: out = x * w / sqrt(mean(x^2) + eps), eps inside the root, the scale multiplies
plainly (src/ops/rmsnorm.rs:38-48).  Statistics in fp32 on the fp32 residual stream."""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..csrc import bindings as B
from ..weights.loader import TensorSpec
from .base import LazyInput, Norm, NormRequest, Runtime, register_part


class ScaledRows(LazyInput):
    """An RMSNorm of the fp32 rows `rows` whose first half is done: `scaled` = bf16(rows * weight) and
    `sumsq` [rows, parts] (partial sums of squares of each row) were written by the kernel that wrote
    `rows`; each row's factor 1 / sqrt(mean + eps) is still to be applied, by the projection that
    reads `scaled` (to its outputs: the product is linear in its input)."""

    def __init__(self, norm: "RMSNorm", rows, scaled, sumsq, parts: int, ctx):
        self.norm, self.rows, self.scaled, self.sumsq, self.parts, self.ctx = norm, rows, scaled, sumsq, parts, ctx

    def row_scale(self) -> B.RowScale:
        return B.RowScale(sumsq=self.sumsq.data_ptr(), parts=self.parts, hidden=self.norm.hidden_size, eps=self.norm.eps)

    def materialize(self, n_rows: int):
        out = self.norm.rt.workspace.take("block.normed", self.rows.shape, self.norm.rt.dtype)
        self.norm.forward(self.rows, out, self.ctx, rows=n_rows)
        return out


def honour(request: NormRequest, rows, ctx, name: str, max_parts: int):
    """For a kernel about to write the fp32 `rows`: the buffers of the norm's first half and the
    kernel argument that names them.  `finish(ahead)` (after the launch) makes the `ScaledRows`."""
    ws = request.norm.rt.workspace
    scaled = ws.take(name + ".ahead_scaled", rows.shape, torch.bfloat16)
    sumsq = ws.take(name + ".ahead_sumsq", (rows.shape[0], max_parts), torch.float32)
    ahead = B.norm_ahead(request.weight, scaled, sumsq)

    def finish():
        return ScaledRows(request.norm, rows, scaled, sumsq, int(ahead.parts), ctx) if ahead.parts > 0 else None
    return ahead, finish


class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, spec, hidden_size: int, rt: Runtime):
        self.eps = float(spec["eps"])
        self.hidden_size = hidden_size
        self.rt = rt
        self.weight = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.hidden_size,), "ones_plus_normal")}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"].contiguous()

    def forward(self, x, out, ctx, rows_idx=None, rows=None) -> None:
        B.rmsnorm(x, self.weight, out, self.eps, ctx.stream, rows_idx=rows_idx, rows=rows)

    def request_ahead(self):
        return NormRequest(self, self.weight, self.eps)


register_part("norm", "rmsnorm", RMSNorm)
