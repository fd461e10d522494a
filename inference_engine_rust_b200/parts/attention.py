"""Grouped-query attention with rotary positions and an optional sliding window, over the
paged cache.

Order of work, as in the reference (src/layers/attention.rs:245-254, 314-352, 364-421 for a
prompt; :518-520, 577-652 for one token): Q/K/V projections, rotate Q and K at the token's
absolute position, store K and V, scores * scale over the visible keys, softmax, weighted
values, output projection, added to the un-normed block input (:757-759).
The three input projections are one product against the row-concatenated matrix
[q_proj; k_proj; v_proj]; its output row is laid out [heads | kv_heads | kv_heads] x head_dim,
which is the layout the rope-and-store and attention kernels index.

A prompt (every sequence starts at position 0) attends over the step's own keys and values;
a one-token step attends over the cache.  An execution that reads another execution's cache
stores nothing and always attends over that cache.
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..cache import KVRequest
from ..csrc import bindings as B
from ..weights.loader import TensorSpec
from .base import Mixer, Runtime, StepContext, part_class, register_part
from .linear import Linear


class Attention(Mixer):
    graph_safe = True
    takes_lazy_input = True          # its input goes to a projection, which may finish a norm itself

    def __init__(self, spec, rt: Runtime):
        self.rt = rt
        self.hidden_size = int(spec["hidden_size"])
        self.heads = int(spec["heads"])
        self.kv_heads = int(spec["kv_heads"])
        self.head_dim = int(spec["head_dim"])
        self.window = spec.get("window")
        self.scale = float(spec["scale"])
        if self.heads % self.kv_heads:
            raise ValueError(f"heads {self.heads} is not a multiple of kv_heads {self.kv_heads}")
        pos = spec["position"]
        self.position = part_class("position", pos.kind)(pos, self.head_dim, rt)
        self.q_dim = self.heads * self.head_dim
        self.kv_dim = self.kv_heads * self.head_dim
        self.qkv = None
        self.o = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        h = self.hidden_size
        specs = {
            "q_proj.weight": TensorSpec((self.q_dim, h)),
            "k_proj.weight": TensorSpec((self.kv_dim, h)),
            "v_proj.weight": TensorSpec((self.kv_dim, h)),
            "o_proj.weight": TensorSpec((h, self.q_dim)),
        }
        # tensors of the position encoding, if it has any, live under "position."
        specs.update({"position." + n: s for n, s in self.position.tensor_specs().items()})
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        dt = self.rt.dtype
        fused = torch.cat([tensors["q_proj.weight"].to(dt), tensors["k_proj.weight"].to(dt),
                           tensors["v_proj.weight"].to(dt)], dim=0)
        self.qkv = Linear(fused, self.rt)
        self.o = Linear(tensors["o_proj.weight"], self.rt)
        self.position.load({n[len("position."):]: t for n, t in tensors.items() if n.startswith("position.")})

    def cache_request(self) -> KVRequest:
        return KVRequest(self.kv_heads, self.head_dim, self.window)

    def weight_bytes(self) -> int:
        return self.qkv.nbytes() + self.o.nbytes()

    def cut_by_length_key(self):
        return ("attention", self.heads, self.kv_heads, self.head_dim, self.window, self.rt.fast)

    def cut_by_length(self, pos0, cache_view) -> bool:
        if not self.rt.fast or cache_view is None:
            return False
        from . import fast_attention
        return fast_attention.wants_length_cut(pos0, self.kv_heads, self.heads // self.kv_heads, self.window,
                                               cache_view.group.page_tokens, self.head_dim)

    def forward(self, xn, residual, ctx: StepContext, cache_view, writes_cache: bool) -> None:
        rt, ws, T = self.rt, self.rt.workspace, ctx.n_tokens
        kv = cache_view.struct
        qkv = ws.take("attn.qkv", (T, self.q_dim + 2 * self.kv_dim), rt.dtype)
        self.qkv.apply(xn, qkv, T, ctx.stream)
        out = ws.take("attn.out", (T, self.q_dim), rt.dtype)
        if rt.fast and ctx.kind == "decode":
            # one token per sequence: rotation, cache write and attention in one kernel, if the
            # position encoding is a plain rotation and the kernel takes the sizes
            from . import fast_attention
            if fast_attention.decode_with_rotation(self, qkv, out, ctx, cache_view, writes_cache):
                self.o.apply(out, residual, T, ctx.stream, add_residual=True, ctx=ctx)
                return
        # positions for queries and keys, then the cache write (the mixer's own business); a plain
        # rotation is fused with the write in one kernel
        rot = getattr(self.position, "rotary_constants", lambda: None)()      # (optional in the interface)
        if rot is not None:
            inv_freq, rotary_dim, pairing = rot
            B.rope_kv_store(qkv, ctx.batch, kv, inv_freq, self.heads, rotary_dim, pairing, writes_cache,
                            rt.err, ctx.stream)
        else:
            self.position.encode(qkv, ctx, self.heads, self.kv_heads)
            if writes_cache:
                B.kv_store(qkv, ctx.batch, kv, self.heads, rt.err, ctx.stream)
        from_cache = ctx.kind == "decode" or not writes_cache
        if from_cache and ctx.kind == "prompt":
            cap = cache_view.group.ring_capacity
            if ctx.max_kv_len > cap:
                raise ValueError(
                    f"a prompt of {ctx.max_kv_len} tokens cannot attend over a shared windowed cache "
                    f"that keeps {cap} positions")
        done = False
        if rt.fast:
            from . import fast_attention
            done = fast_attention.apply(self, qkv, out, ctx, cache_view, from_cache)
        if not done:
            B.attention_plain(qkv, out, ctx.batch, kv, self.heads, self.scale, from_cache,
                              rt.err, ctx.stream)
        self.o.apply(out, residual, T, ctx.stream, add_residual=True, ctx=ctx)


register_part("mixer", "attention", Attention)
