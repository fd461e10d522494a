"""Dispatch of attention to the fast kernels (flash prompt attention, split-KV decode)."""
from __future__ import annotations

import os

import torch

from ..csrc import bindings as B

_CTAS_PER_SM = 2                 # two CTAs fit an SM (three-page rings of keys and values)
_MAX_SPLITS = 16


def decode_splits(n_tokens: int, kv_heads: int, group: int) -> int:
    """How many ways the keys of each sequence are split: enough CTAs to fill the GPU at
    small batches, one split once the batch alone does.  Depends on the (padded) batch size
    only, never on the sequences' lengths, so a captured graph stays valid."""
    slices = -(-group // 8)
    ctas = max(1, n_tokens * kv_heads * slices)
    return max(1, min(_MAX_SPLITS, _CTAS_PER_SM * B.sm_count() // ctas))      # as many splits as stay one wave


def decode_with_rotation(attn, qkv, out, ctx, cache_view, writes_cache: bool) -> bool:
    """One-token step with the rotary encoding and the cache write inside the attention kernel.
    False (nothing launched) if the position encoding is no plain rotation or the kernel does
    not take this cache; the caller then encodes, stores and attends in separate kernels."""
    rot = attn.position.rotary_constants()
    if rot is None or qkv.dtype != torch.bfloat16 or os.environ.get("IERT_FUSED_ROPE", "1") == "0":
        return False
    inv_freq, rotary_dim, pairing = rot
    rt = attn.rt
    splits = decode_splits(ctx.n_tokens, attn.kv_heads, attn.heads // attn.kv_heads)
    n = B.attention_decode_scratch_floats(ctx.n_tokens, attn.heads, attn.head_dim, splits)
    scratch = rt.workspace.take("attn.decode_scratch", (n,), torch.float32)
    return B.attention_decode_tc_rope(qkv, out, ctx.batch, cache_view.struct, attn.heads, attn.scale, splits,
                                      scratch, inv_freq, rotary_dim, pairing, writes_cache, rt.err, ctx.stream)


def apply(attn, qkv, out, ctx, cache_view, from_cache: bool) -> bool:
    """Run a fast kernel if one takes this case; False means the caller runs the plain one."""
    rt = attn.rt
    if qkv.dtype != torch.bfloat16:
        return False
    if ctx.kind == "decode":
        splits = decode_splits(ctx.n_tokens, attn.kv_heads, attn.heads // attn.kv_heads)
        n = B.attention_decode_scratch_floats(ctx.n_tokens, attn.heads, attn.head_dim, splits)
        scratch = rt.workspace.take("attn.decode_scratch", (n,), torch.float32)
        if B.attention_decode_tc(qkv, out, ctx.batch, cache_view.struct, attn.heads, attn.scale, splits,
                                 scratch, rt.err, ctx.stream):
            return True
        return B.attention_decode(qkv, out, ctx.batch, cache_view.struct, attn.heads, attn.scale, splits,
                                  scratch, rt.err, ctx.stream)
    if not from_cache:
        return B.attention_prefill(qkv, out, ctx.batch, attn.heads, attn.kv_heads, attn.head_dim,
                                   attn.window or 0, attn.scale, ctx.max_q_len, ctx.stream, err=rt.err)
    return False
