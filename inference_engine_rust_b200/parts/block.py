"""Arrangement of a layer's parts.  "prenorm": x += mixer(norm1(x)); x += ffn(norm2(x)) (the second
half left out for a layer without a feed-forward)
(src/layers/block.rs:19-24,63-65; the residual uses the un-normed input,
src/layers/attention.rs:757-759, src/layers/ffn.rs:113-116)."""
from __future__ import annotations

from .base import Block, Runtime, StepContext, first_norm_request_of, register_part


class PreNormBlock(Block):
    graph_safe = True

    def __init__(self, layer_spec, norm1, mixer, norm2, ffn, rt: Runtime):
        self.norm1, self.mixer, self.norm2, self.ffn, self.rt = norm1, mixer, norm2, ffn, rt

    def forward(self, x, ctx: StepContext, cache_view, writes_cache: bool) -> None:
        xn = self._normed(self.norm1, x, ctx)
        # what the next norm asks of whoever adds the mixer's result into x
        if self.ffn is not None:
            ctx.norm_ahead = self._request(self.norm2, self.ffn, ctx)
        else:
            ctx.norm_ahead = first_norm_request_of(ctx.next_block, ctx)
        self.mixer.forward(xn, x, ctx, cache_view, writes_cache)
        if self.ffn is None:                     # a layer without a feed-forward
            ctx.norm_ahead = None
            return
        xn = self._normed(self.norm2, x, ctx)
        ctx.norm_ahead = first_norm_request_of(ctx.next_block, ctx)
        self.ffn.forward(xn, x, ctx)
        ctx.norm_ahead = None

    def first_norm_request(self, ctx: StepContext):
        return self._request(self.norm1, self.mixer, ctx)

    def _request(self, norm, part, ctx: StepContext):
        """In steps of up to 64 tokens (one-token steps, short prompts) a norm may ask whoever writes its
        input rows to do its element-wise half (`NormRequest`), if the part behind it hands its input to a
        projection."""
        from . import fast_linear
        if (self.rt.fast and ctx.n_tokens <= fast_linear.NORM_AHEAD_MAX_TOKENS
                and getattr(part, "takes_lazy_input", False) and fast_linear.norm_ahead_enabled()):
            return norm.request_ahead()
        return None

    def _normed(self, norm, x, ctx: StepContext):
        """norm(x): what the writer of x left behind for this norm, if it honoured the norm's request,
        else the norm's own kernel."""
        lazy, ctx.rows_ahead = ctx.rows_ahead, None
        if lazy is not None and getattr(lazy, "norm", None) is norm and lazy.rows is x:
            return lazy
        xn = self.rt.workspace.take("block.normed", x.shape, self.rt.dtype)
        norm.forward(x, xn, ctx, rows=ctx.n_tokens)
        return xn


register_part("block", "prenorm", PreNormBlock)
