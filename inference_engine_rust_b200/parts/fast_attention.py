"""Dispatch of attention to the fast kernels (flash prompt attention, split-KV decode)."""
from __future__ import annotations


def apply(attn, qkv, out, ctx, cache_view, from_cache: bool) -> bool:
    """Run a fast kernel if one takes this case; False means the caller runs the plain one."""
    return False
