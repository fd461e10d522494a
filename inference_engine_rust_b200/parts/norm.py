"""RMSNorm: out = x * w / sqrt(mean(x^2) + eps), eps inside the root, the scale multiplies
plainly (src/ops/rmsnorm.rs:38-48).  Statistics in fp32 on the fp32 residual stream."""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..csrc import bindings as B
from ..weights.loader import TensorSpec
from .base import Norm, Runtime, register_part


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


register_part("norm", "rmsnorm", RMSNorm)
