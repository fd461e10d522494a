"""Arrangement of a layer's parts.  "prenorm": x += mixer(norm1(x)); x += ffn(norm2(x))
(src/layers/block.rs:19-24,63-65; the residual uses the un-normed input,
src/layers/attention.rs:757-759, src/layers/ffn.rs:113-116)."""
from __future__ import annotations

from .base import Block, Runtime, StepContext, register_part


class PreNormBlock(Block):
    graph_safe = True

    def __init__(self, layer_spec, norm1, mixer, norm2, ffn, rt: Runtime):
        self.norm1, self.mixer, self.norm2, self.ffn, self.rt = norm1, mixer, norm2, ffn, rt

    def forward(self, x, ctx: StepContext, cache_view, writes_cache: bool) -> None:
        xn = self.rt.workspace.take("block.normed", x.shape, self.rt.dtype)
        self.norm1.forward(x, xn, ctx, rows=ctx.n_tokens)
        self.mixer.forward(xn, x, ctx, cache_view, writes_cache)
        self.norm2.forward(x, xn, ctx, rows=ctx.n_tokens)
        self.ffn.forward(xn, x, ctx)


register_part("block", "prenorm", PreNormBlock)
