"""Dispatch of attention to the fast kernels (flash prompt attention, split-KV decode)."""
from __future__ import annotations

import os

import torch

from ..csrc import bindings as B

def _slots(head_dim: int) -> int:
    """CTAs of the split-KV decode kernel that the device holds at once (how many an SM holds is a
    fact of that kernel, asked of its library; the CUDA-core kernel for other head sizes is
    given the same rule)."""
    per_sm = B.attention_decode_ctas_per_sm(head_dim) if head_dim % 16 == 0 and 16 <= head_dim <= 256 else 2
    return per_sm * B.sm_count()


_MAX_SPLITS = 16


def decode_splits(n_tokens: int, kv_heads: int, group: int, head_dim: int) -> int:
    """How many ways the keys of each sequence are split: enough CTAs to fill the GPU at
    small batches, one split once the batch alone does.  Depends on the (padded) batch size
    only, never on the sequences' lengths, so a captured graph stays valid."""
    slices = -(-group // 8)
    ctas = max(1, n_tokens * kv_heads * slices)
    return max(1, min(_MAX_SPLITS, _slots(head_dim) // ctas))      # as many splits as stay one wave


def wants_length_cut(pos0, kv_heads: int, group: int, window, page_tokens: int, head_dim: int) -> bool:
    """Should a one-token step over sequences at these positions be cut by length (see
    `decode_parts`) rather than evenly?  Yes if the longest sequence reads over 1.3 times the
    average number of pages (an even cut ends when its CTAs do).  And yes if the batch alone
    fills the device and a cut by length is predicted to take at least 15 % fewer page loads
    in a row: 48 sequences of 33 pages with 8 kv heads are 384 CTAs on 296 slots, two rounds
    of 33 pages; cut in two they are 768 CTAs, three rounds of 17."""
    n = len(pos0)
    if n < 2:
        return False
    if window:
        pages = [p // page_tokens + 1 - max(0, p + 1 - window) // page_tokens for p in pos0]
    else:
        pages = [p // page_tokens + 1 for p in pos0]
    longest, total = max(pages), sum(pages)
    if longest * n > 1.3 * total:
        return True
    per_sequence = kv_heads * -(-group // 8)
    slots = _slots(head_dim)
    if n * per_sequence <= slots:
        return False
    even = -(-n * per_sequence // slots) * longest
    per_part = max(1, -(-total * per_sequence // (2 * slots)))                 # as the kernel works it out
    parts = [min(8, -(-p // per_part)) for p in pages]
    cut = -(-sum(parts) * per_sequence // slots) * max(-(-p // k) for p, k in zip(pages, parts))
    return even >= 1.15 * cut


def decode_parts(n_tokens: int, kv_heads: int, group: int, unequal: bool, head_dim: int):
    """(most parts a sequence is cut into, CTAs to aim for) for the tensor-core decode kernel.  With
    sequences of unequal lengths (the engine's hint) a long sequence is cut into more parts than a
    short one, up to four times the even split, so that all CTAs hold about the same number of
    pages: how many parts each sequence gets is worked out on the device from the lengths, which
    costs a few microseconds that steps of equal lengths do not spend (target 0: every sequence
    into all parts).  Both numbers depend on the (padded) batch size and the hint only."""
    base = decode_splits(n_tokens, kv_heads, group, head_dim)
    if not unequal or os.environ.get("IERT_DECODE_BALANCE", "1") == "0":
        return base, 0
    ctas = max(1, n_tokens * kv_heads * -(-group // 8))
    if base < 2:
        # the batch alone fills the device: aim for two rounds of CTA slots, so that a sequence of
        # about average length stays whole or is cut in two and one that is k times longer into
        # about k parts (at most 8), or its single CTA would end the step alone
        return 8, 2 * _slots(head_dim)
    return min(_MAX_SPLITS, 4 * base), base * ctas


def decode_with_rotation(attn, qkv, out, ctx, cache_view, writes_cache: bool) -> bool:
    """One-token step with the rotary encoding and the cache write inside the attention kernel.
    False (nothing launched) if the position encoding is no plain rotation or the kernel does
    not take this cache; the caller then encodes, stores and attends in separate kernels."""
    rot = getattr(attn.position, "rotary_constants", lambda: None)()
    if rot is None or qkv.dtype != torch.bfloat16 or os.environ.get("IERT_FUSED_ROPE", "1") == "0":
        return False
    inv_freq, rotary_dim, pairing = rot
    rt = attn.rt
    parts, target = decode_parts(ctx.n_tokens, attn.kv_heads, attn.heads // attn.kv_heads, ctx.unequal_lengths, attn.head_dim)
    n = B.attention_decode_scratch_floats(ctx.n_tokens, attn.heads, attn.head_dim, parts)
    scratch = rt.workspace.take("attn.decode_scratch", (n,), torch.float32)
    return B.attention_decode_tc_rope(qkv, out, ctx.batch, cache_view.struct, attn.heads, attn.scale, parts,
                                      scratch, inv_freq, rotary_dim, pairing, writes_cache, rt.err, ctx.stream,
                                      target_ctas=target)


def apply(attn, qkv, out, ctx, cache_view, from_cache: bool) -> bool:
    """Run a fast kernel if one takes this case; False means the caller runs the plain one."""
    rt = attn.rt
    if qkv.dtype != torch.bfloat16:
        return False
    if ctx.kind == "decode":
        splits = decode_splits(ctx.n_tokens, attn.kv_heads, attn.heads // attn.kv_heads, attn.head_dim)
        parts, target = decode_parts(ctx.n_tokens, attn.kv_heads, attn.heads // attn.kv_heads, ctx.unequal_lengths, attn.head_dim)
        n = B.attention_decode_scratch_floats(ctx.n_tokens, attn.heads, attn.head_dim, max(parts, splits))
        scratch = rt.workspace.take("attn.decode_scratch", (n,), torch.float32)
        if B.attention_decode_tc(qkv, out, ctx.batch, cache_view.struct, attn.heads, attn.scale, parts,
                                 scratch, rt.err, ctx.stream, target_ctas=target):
            return True
        return B.attention_decode(qkv, out, ctx.batch, cache_view.struct, attn.heads, attn.scale, splits,
                                  scratch, rt.err, ctx.stream)
    if not from_cache:
        return B.attention_prefill(qkv, out, ctx.batch, attn.heads, attn.kv_heads, attn.head_dim,
                                   attn.window or 0, attn.scale, ctx.max_q_len, ctx.stream, err=rt.err)
    return False
