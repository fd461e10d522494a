"""Dense gated feed-forward: y = (silu(x Wg^T) * (x Wu^T)) Wd^T, added to the block input
(src/layers/ffn.rs:35-63,113-116; src/ops/swiglu.rs:3-36).  Gate and up are one product
against the row-concatenated matrix [gate_proj; up_proj]: output columns [0, I) are the
gate, [I, 2I) the up projection, which is what the activation kernel indexes."""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..csrc import bindings as B
from ..weights.loader import TensorSpec
from .base import FeedForward, Runtime, StepContext, register_part
from .linear import Linear


class SwiGLU(FeedForward):
    graph_safe = True
    takes_lazy_input = True          # its input goes to a projection, which may finish a norm itself

    def __init__(self, spec, rt: Runtime):
        self.rt = rt
        self.hidden_size = int(spec["hidden_size"])
        self.intermediate_size = int(spec["intermediate_size"])
        self.gate_up = None
        self.down = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        h, i = self.hidden_size, self.intermediate_size
        return {
            "gate_proj.weight": TensorSpec((i, h)),
            "up_proj.weight": TensorSpec((i, h)),
            "down_proj.weight": TensorSpec((h, i)),
        }

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        dt = self.rt.dtype
        fused = torch.cat([tensors["gate_proj.weight"].to(dt), tensors["up_proj.weight"].to(dt)], dim=0)
        self.gate_up = Linear(fused, self.rt)
        self.down = Linear(tensors["down_proj.weight"], self.rt)

    def weight_bytes(self) -> int:
        return self.gate_up.nbytes() + self.down.nbytes()

    def forward(self, xn, residual, ctx: StepContext) -> None:
        rt, ws, T, I = self.rt, self.rt.workspace, ctx.n_tokens, self.intermediate_size
        act = ws.take("ffn.act", (T, I), rt.dtype)
        done = False
        if rt.fast:
            from . import fast_linear
            done = fast_linear.apply_gated(self.gate_up, xn, act, T, ctx.stream)
        if not done:
            gu = ws.take("ffn.gate_up", (T, 2 * I), rt.dtype)
            self.gate_up.apply(xn, gu, T, ctx.stream)
            B.silu_mul(gu, act, T, I, ctx.stream)
        self.down.apply(act, residual, T, ctx.stream, add_residual=True, ctx=ctx)


register_part("ffn", "swiglu", SwiGLU)
