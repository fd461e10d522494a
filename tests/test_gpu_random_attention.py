"""The attention kernels on batches drawn at random, against the plain kernel (one block per token and
head, float32 arithmetic): decode attention over caches of unequal lengths with random head shapes,
windows, numbers of parts and ways of cutting; prompt attention over packed prompts of random lengths."""
import math
import os

import numpy as np
import pytest
import torch

from test_gpu_kernels import B, DEV, err_word, make_batch, make_cache, stream

pytestmark = pytest.mark.gpu
N_CASES = int(os.environ.get("IERT_TEST_RANDOM_ATTENTION", "10"))     # (more for a longer hunt)
SHAPES = [(32, 8, 128), (8, 8, 64), (6, 2, 32), (5, 1, 80), (16, 2, 128), (4, 4, 256), (3, 3, 48), (12, 4, 96)]


def draw_decode(rng):
    heads, kvh, hd = SHAPES[int(rng.integers(0, len(SHAPES)))]
    n = int(rng.choice([1, 2, 5, 8, 17, 33, 64]))
    longest = int(rng.choice([70, 300, 1500, 5000 if n <= 8 else 700]))
    lens = [int(x) for x in rng.integers(1, longest + 1, n)]
    window = rng.choice([None, 16, 70, 1000])
    parts = int(rng.choice([1, 2, 4, 8, 16]))
    target = int(rng.choice([0, 64, 296, 600]))
    return heads, kvh, hd, lens, None if window is None else int(window), parts, target


DECODE_CASES = [draw_decode(np.random.default_rng(900 + i)) for i in range(N_CASES)]


@pytest.mark.parametrize("heads,kvh,hd,lens,window,parts,target", DECODE_CASES,
                         ids=[f"h{c[0]}x{c[1]}d{c[2]}-n{len(c[3])}-max{max(c[3])}-W{c[4]}-p{c[5]}-t{c[6]}" for c in DECODE_CASES])
def test_decode_attention_on_a_random_batch(heads, kvh, hd, lens, window, parts, target):
    b = B()
    g = torch.Generator(device=DEV).manual_seed(sum(lens) + heads)
    dtype = torch.bfloat16
    pages = sum(-(-n // 64) for n in lens)
    cache = make_cache(kvh, hd, window, dtype, max_tokens=64 * pages, max_seq_len=64 * -(-max(lens) // 64), slots=len(lens))
    slots = [cache.open_sequence() for _ in lens]
    for s_, n in zip(slots, lens):
        cache.reserve(s_, n)
    cache.upload()
    kvs = cache.layer_view(0).struct
    W = heads + 2 * kvh
    scale = 1.0 / math.sqrt(hd)
    ident = torch.zeros(hd // 2, device=DEV)
    err = err_word()
    fill = (torch.randn(sum(n - 1 for n in lens), W * hd, device=DEV, generator=g) * 0.7).to(dtype)
    nxt = (torch.randn(len(lens), W * hd, device=DEV, generator=g) * 0.7).to(dtype)
    multi = [(s_, n) for s_, n in zip(slots, lens) if n > 1]
    if multi:
        view, keep = make_batch([n - 1 for _, n in multi], [0] * len(multi), [s_ for s_, _ in multi])
        b.rope_kv_store(fill, view, kvs, ident, heads, hd, b.PAIR_HALF, True, err, stream())
    view1, keep1 = make_batch([1] * len(lens), [n - 1 for n in lens], slots)
    b.rope_kv_store(nxt, view1, kvs, ident, heads, hd, b.PAIR_HALF, True, err, stream())
    plain = torch.empty(len(lens), heads * hd, device=DEV, dtype=dtype)
    b.attention_plain(nxt, plain, view1, kvs, heads, scale, True, err, stream())
    n_s = b.attention_decode_scratch_floats(len(lens), heads, hd, parts)
    scratch = torch.full((n_s,), float("nan"), device=DEV)
    tc = torch.full_like(plain, float("nan"))
    assert b.attention_decode_tc(nxt, tc, view1, kvs, heads, scale, parts, scratch, err, stream(), target_ctas=target)
    torch.cuda.synchronize()
    assert err.item() == 0, b.describe_error_bits(err.item())
    assert torch.isfinite(tc).all()
    assert torch.allclose(tc.float(), plain.float(), atol=2e-2, rtol=2e-2), \
        f"max diff {(tc.float() - plain.float()).abs().max().item():.4g}"
    if hd % 8 == 0 and target == 0:          # the CUDA-core sibling, cut evenly
        scratch.fill_(float("nan"))
        cc = torch.full_like(plain, float("nan"))
        if b.attention_decode(nxt, cc, view1, kvs, heads, scale, parts, scratch, err, stream()):
            torch.cuda.synchronize()
            assert err.item() == 0
            assert torch.allclose(cc.float(), plain.float(), atol=2e-2, rtol=2e-2)


def draw_prompt(rng):
    heads, kvh, hd = SHAPES[int(rng.integers(0, len(SHAPES)))]
    n = int(rng.integers(1, 6))
    q_lens = [int(rng.choice([1, 2, 31, 63, 64, 65, 127, 128, 129, 200, 333, 700])) for _ in range(n)]
    window = rng.choice([None, 1, 16, 70, 129, 400])
    return heads, kvh, hd, q_lens, None if window is None else int(window)


PROMPT_CASES = [draw_prompt(np.random.default_rng(950 + i)) for i in range(N_CASES)]


@pytest.mark.parametrize("heads,kvh,hd,q_lens,window", PROMPT_CASES,
                         ids=[f"h{c[0]}x{c[1]}d{c[2]}-q{'_'.join(map(str, c[3]))}-W{c[4]}" for c in PROMPT_CASES])
def test_prompt_attention_on_random_prompts(heads, kvh, hd, q_lens, window):
    b = B()
    g = torch.Generator(device=DEV).manual_seed(sum(q_lens) + heads)
    dtype = torch.bfloat16
    T, W = sum(q_lens), heads + 2 * kvh
    scale = 1.0 / math.sqrt(hd)
    cache = make_cache(kvh, hd, window, dtype, slots=len(q_lens))            # only its geometry is used
    view, keep = make_batch(q_lens, [0] * len(q_lens), list(range(len(q_lens))))
    qkv = (torch.randn(T, W * hd, device=DEV, generator=g) * 0.7).to(dtype)
    err = err_word()
    plain = torch.empty(T, heads * hd, device=DEV, dtype=dtype)
    b.attention_plain(qkv, plain, view, cache.layer_view(0).struct, heads, scale, False, err, stream())
    for legacy in (True, False):
        fast = torch.full_like(plain, float("nan"))
        assert b.attention_prefill(qkv, fast, view, heads, kvh, hd, window or 0, scale, max(q_lens), stream(),
                                   err=err, legacy=legacy)
        torch.cuda.synchronize()
        assert err.item() == 0, b.describe_error_bits(err.item())
        assert torch.isfinite(fast).all()
        assert torch.allclose(fast.float(), plain.float(), atol=2e-2, rtol=2e-2), \
            f"legacy={legacy}: max diff {(fast.float() - plain.float()).abs().max().item():.4g}"
