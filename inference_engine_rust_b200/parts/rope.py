"""Rotary position encoding as a part: its constants (theta, how many dimensions rotate,
which elements pair up) are parameters; a mixer's kernel may apply the rotation itself
(`rotary_constants`: fused with its cache write, or with its attention in one-token steps).

angle(pos, k) = pos * theta^(-2k / rotary_dim), computed in fp32 on the device from a
table of theta^(-2k / rotary_dim) made here in double precision.  (The reference reaches
the same angle by repeated fp32 multiplication, src/ops/rope.rs:40-57; the two differ by
that loop's rounding only.)  Pairing "interleaved" rotates (2k, 2k+1) as the reference
does on its row-permuted tensors; "half" rotates (k, k + rotary_dim/2), which is the same
rotation on tensors in safetensors row order (src/layers/attention.rs:137-172).
"""
from __future__ import annotations

import torch

from ..csrc import bindings as B
from .base import PositionEncoding, Runtime, register_part

PAIRINGS = {"half": B.PAIR_HALF, "interleaved": B.PAIR_INTERLEAVED}


class RotaryEncoding(PositionEncoding):
    def __init__(self, spec, head_dim: int, rt: Runtime):
        self.theta = float(spec["theta"])
        self.head_dim = head_dim
        self.rotary_dim = int(spec.get("rotary_dim", head_dim))
        pairing = spec.get("pairing", "half")
        if pairing not in PAIRINGS:
            raise ValueError(f"rope pairing must be one of {sorted(PAIRINGS)}, got {pairing!r}")
        if self.rotary_dim % 2 or not 0 <= self.rotary_dim <= head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {head_dim}")
        self.pairing = PAIRINGS[pairing]
        k = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
        inv = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * k / max(self.rotary_dim, 1))
        factors = spec.get("freq_factors")       # optional per-pair divisors (src/ops/rope.rs:45-50)
        if factors is not None:
            inv = inv / torch.as_tensor(factors, dtype=torch.float64)
        self.inv_freq = inv.to(torch.float32).to(rt.device)

    def rotary_constants(self):
        return self.inv_freq, self.rotary_dim, self.pairing

    def encode(self, qkv, ctx, heads: int, kv_heads: int) -> None:
        B.rotate_qk(qkv, ctx.batch, self.inv_freq, heads, kv_heads, self.head_dim, self.rotary_dim, self.pairing,
                    ctx.rt.err, ctx.stream)


register_part("position", "rope", RotaryEncoding)
