"""The output head: logits = hn . W^T over the whole vocabulary, in float32.

Reference: the last row through `output.weight` (src/engine/runtime.rs:76-116); tied to the
embedding table when the file has no such tensor (src/model_weights/names.rs:300-310), which the
model decides when it loads.  Registered as head kind "linear"; another head (logits with a soft
cap, a scale, a bias) registers under its own kind and is named by `ModelSpec.head`.
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..config.specs import PartSpec
from ..weights.loader import TensorSpec
from .base import Head, Runtime, StepContext, register_part
from .linear import Linear


class LinearHead(Head):
    graph_safe = True

    def __init__(self, spec: PartSpec, hidden_size: int, vocab_size: int, rt: Runtime):
        self.hidden_size, self.vocab_size, self.rt = hidden_size, vocab_size, rt
        self.proj = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.vocab_size, self.hidden_size))}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.proj = Linear(tensors["weight"], self.rt)

    @property
    def weight(self) -> torch.Tensor:
        return self.proj.weight

    def nbytes(self) -> int:
        return self.proj.nbytes()

    def forward(self, hn, logits, n_rows: int, ctx: StepContext) -> None:
        self.proj.apply(hn, logits, n_rows, ctx.stream)


register_part("head", "linear", LinearHead)
