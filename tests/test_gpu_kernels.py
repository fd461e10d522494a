"""Each kernel alone against a plain PyTorch float32 statement of the same operation, at
sizes other than the tiny models': widths and vocabularies that are no power of two, head
sizes in steps of 16, odd numbers of heads and groups."""
import math

import numpy as np
import pytest
import torch

from plain import mistral_plain as P

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def B():
    from inference_engine_rust_b200.csrc import bindings
    return bindings


def stream():
    return B().stream_ptr()


def err_word():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


def make_batch(q_lens, pos0, slots):
    """Device arrays and the BatchView of a step with these sequences."""
    b = B()
    n, T = len(q_lens), sum(q_lens)
    cu = np.zeros(n + 1, dtype=np.int32)
    cu[1:] = np.cumsum(q_lens)
    tok_seq = np.repeat(np.arange(n, dtype=np.int32), q_lens)
    arrs = [torch.tensor(a, dtype=torch.int32, device=DEV) for a in (cu, slots, tok_seq, pos0)]
    view = b.BatchView(cu_q=arrs[0].data_ptr(), slot_ids=arrs[1].data_ptr(), tok_seq=arrs[2].data_ptr(),
                       pos0=arrs[3].data_ptr(), n_seqs=n, n_tokens=T)
    return view, arrs


def make_cache(kv_heads, head_dim, window, dtype, max_tokens=64 * 16, max_seq_len=640, slots=4):
    from inference_engine_rust_b200.cache import Cache, KVRequest
    return Cache({0: KVRequest(kv_heads, head_dim, window)}, max_tokens=max_tokens, max_seq_len=max_seq_len,
                 max_sequences=slots, dtype=dtype, device=DEV, poison=True)


# ---------------------------------------------------------------------------------------


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed_gather(dtype):
    torch.manual_seed(0)
    table = torch.randn(331, 88, device=DEV).to(dtype)
    ids = torch.tensor([0, 330, 17, 17, 5], dtype=torch.int32, device=DEV)
    x = torch.empty(5, 88, device=DEV)
    err = err_word()
    B().embed_gather(table, ids, x, 1.5, err, stream())
    assert torch.equal(x, table[ids.long()].float() * 1.5) and err.item() == 0
    bad = torch.tensor([3, 331, -1], dtype=torch.int32, device=DEV)
    x3 = torch.empty(3, 88, device=DEV)
    B().embed_gather(table, bad, x3, 1.0, err, stream())
    assert err.item() == B().ERR_TOKEN_RANGE and float(x3[1:].abs().sum()) == 0


@pytest.mark.parametrize("hidden", [88, 1000, 4104])
@pytest.mark.parametrize("wdt,odt", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                     (torch.float32, torch.bfloat16)])
def test_rmsnorm(hidden, wdt, odt):
    torch.manual_seed(1)
    x = torch.randn(7, hidden, device=DEV) * 3
    w = (1 + 0.1 * torch.randn(hidden, device=DEV)).to(wdt)
    out = torch.empty(7, hidden, device=DEV, dtype=odt)
    B().rmsnorm(x, w, out, 1e-5, stream())
    ref = P.rmsnorm(x.cpu(), w.float().cpu(), 1e-5)
    tol = 1e-5 if odt == torch.float32 else 1e-2
    assert torch.allclose(out.float().cpu(), ref, atol=tol, rtol=tol)
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    out2 = torch.empty(3, hidden, device=DEV, dtype=odt)
    B().rmsnorm(x, w, out2, 1e-5, stream(), rows_idx=rows)
    assert torch.equal(out2, out[rows.long()])


@pytest.mark.parametrize("M,N,K", [(1, 53, 71), (37, 53, 71), (130, 200, 96), (5, 331, 88)])
def test_gemm_plain(M, N, K):
    torch.manual_seed(2)
    x = torch.randn(M, K, device=DEV)
    w = torch.randn(N, K, device=DEV)
    out = torch.empty(M, N, device=DEV)
    b = B()
    b.gemm_plain(x, w, out, M, b.GEMM_STORE, stream())
    ref = (x.double() @ w.double().t()).float()
    assert torch.allclose(out, ref, atol=1e-4, rtol=1e-5)
    res = torch.randn(M, N, device=DEV)
    res0 = res.clone()
    b.gemm_plain(x, w, res, M, b.GEMM_ADD_RESIDUAL, stream())
    assert torch.allclose(res, res0 + ref, atol=1e-4, rtol=1e-5)
    xb, wb = x.bfloat16(), w.bfloat16()
    outb = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    b.gemm_plain(xb, wb, outb, M, b.GEMM_STORE, stream())
    refb = (xb.double() @ wb.double().t()).float()
    assert torch.allclose(outb.float(), refb, atol=0.1, rtol=1e-2)
    # one row's result does not depend on how many rows the call has
    one = torch.empty(1, N, device=DEV)
    b.gemm_plain(x[M - 1:], w, one, 1, b.GEMM_STORE, stream())
    assert torch.equal(one[0], out[M - 1])


def test_silu_mul():
    torch.manual_seed(3)
    gu = torch.randn(9, 2 * 200, device=DEV) * 4
    gu[0, 0], gu[0, 1] = -120.0, 120.0
    out = torch.empty(9, 200, device=DEV)
    B().silu_mul(gu, out, 9, 200, stream())
    ref = P.swiglu(gu[:, :200].cpu(), gu[:, 200:].cpu())
    assert torch.allclose(out.cpu(), ref, atol=1e-6, rtol=1e-5) and torch.isfinite(out).all()
    gb = gu.bfloat16()
    ob = torch.empty(9, 200, device=DEV, dtype=torch.bfloat16)
    B().silu_mul(gb, ob, 9, 200, stream())
    refb = P.swiglu(gb[:, :200].float().cpu(), gb[:, 200:].float().cpu())
    assert torch.allclose(ob.float().cpu(), refb, atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("pairing,rotary", [("half", 48), ("interleaved", 48), ("half", 32)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rope_and_cache_write(pairing, rotary, dtype):
    """Rotation at each token's own position and the write into the right page row, for a
    prompt longer than the ring and for single tokens at large positions."""
    from inference_engine_rust_b200.parts.rope import RotaryEncoding
    from inference_engine_rust_b200.parts.base import Runtime
    from inference_engine_rust_b200.config.specs import PartSpec
    b = B()
    heads, kvh, hd, theta, window = 3, 3, 48, 50000.0, 70
    cache = make_cache(kvh, hd, window, dtype)
    g = cache.kv_groups[0]
    assert g.ring_pages == 2
    rt = Runtime(dtype=dtype, device=DEV)
    rope = RotaryEncoding(PartSpec("rope", {"theta": theta, "rotary_dim": rotary, "pairing": pairing}), hd, rt)
    torch.manual_seed(4)
    for q_lens, pos0 in (([150, 5], [0, 0]), ([1, 1], [150, 5]), ([1], [437])):
        slots = [cache.open_sequence() for _ in q_lens]
        for s, p, q in zip(slots, pos0, q_lens):
            cache.reserve(s, p + q)
        cache.upload()
        view, keep = make_batch(q_lens, pos0, slots)
        T = sum(q_lens)
        qkv = torch.randn(T, (heads + 2 * kvh) * hd, device=DEV).to(dtype)
        before = qkv.float().cpu().view(T, heads + 2 * kvh, hd)
        err = err_word()
        b.rope_kv_store(qkv, view, cache.layer_view(0).struct, rope.inv_freq, heads, rotary,
                        rope.pairing, True, err, stream())
        assert err.item() == 0
        after = qkv.float().cpu().view(T, heads + 2 * kvh, hd)
        kc, vc = g.k[0].float().cpu(), g.v[0].float().cpu()
        # the plain angle is formed by k repeated fp32 multiplications (relative error about
        # k * 2^-24), the kernel's by one: at position ~440 they differ by up to ~5e-5 rad
        tol = 1e-4 if dtype == torch.float32 else 2e-2
        t = 0
        for s, p0, q in zip(slots, pos0, q_lens):
            for i in range(q):
                pos = p0 + i
                for h in range(heads + kvh):
                    ref = P.rope(before[t, h], theta, pos, hd, rotary, pairing)
                    assert torch.allclose(after[t, h], ref, atol=tol, rtol=tol), (pos, h)
                assert torch.equal(after[t, heads + kvh:], before[t, heads + kvh:])      # values untouched
                stored = pos >= p0 + q - g.ring_capacity
                page = g.pages_of(s)[(pos // 64) % g.ring_pages]
                if stored:
                    assert torch.equal(kc[page, :, pos % 64], after[t, heads:heads + kvh])
                    assert torch.equal(vc[page, :, pos % 64], before[t, heads + kvh:])
                t += 1
        for s in slots:
            cache.close_sequence(s)


def _plain_attention(q, k, v, heads, kvh, scale, window):
    """q [Tq, heads, hd] at positions Tk-Tq..Tk-1 over keys k, v [Tk, kvh, hd]."""
    Tq, Tk = q.shape[0], k.shape[0]
    out = torch.zeros_like(q)
    for i in range(Tq):
        pos = Tk - Tq + i
        lo = max(0, pos - (window - 1)) if window else 0
        for h in range(heads):
            kh = h // (heads // kvh)
            s = (k[lo:pos + 1, kh] @ q[i, h]) * scale
            out[i, h] = P.softmax(s) @ v[lo:pos + 1, kh]
    return out


@pytest.mark.parametrize("heads,kvh,hd,window", [(4, 2, 16, 16), (6, 1, 32, None), (3, 3, 48, 70),
                                                 (8, 2, 128, None), (5, 5, 80, 33)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_plain_prompt_and_cache(heads, kvh, hd, window, dtype):
    """Prompts of unequal lengths over their own keys; then one more token each over the
    cache; both against per-row softmax attention.  One query and one far key are scaled up
    so that a single score among hundreds decides the output."""
    b = B()
    torch.manual_seed(5)
    cache = make_cache(kvh, hd, window, dtype)
    g = cache.kv_groups[0]
    q_lens = [300, 1, 77]
    slots = [cache.open_sequence() for _ in q_lens]
    for s, q in zip(slots, q_lens):
        cache.reserve(s, q + 1)
    cache.upload()
    T = sum(q_lens)
    W = heads + 2 * kvh
    scale = 1.0 / math.sqrt(hd)
    qkv = (torch.randn(T, W, hd, device=DEV) * 0.7)
    qkv[299, :heads] *= 4.0                       # the last query of request 0 ...
    far = 299 - (window - 1) if window else 0     # ... and the farthest key it may see
    qkv[far, heads:heads + kvh] = qkv[299, :kvh * (heads // kvh):heads // kvh] * 1.0
    qkv = qkv.to(dtype).view(T, W * hd)
    ident = torch.zeros(hd // 2, device=DEV)      # angle 0: store without rotating
    view, keep = make_batch(q_lens, [0, 0, 0], slots)
    err = err_word()
    b.rope_kv_store(qkv, view, cache.layer_view(0).struct, ident, heads, hd, b.PAIR_HALF, True, err, stream())
    out = torch.empty(T, heads * hd, device=DEV, dtype=dtype)
    b.attention_plain(qkv, out, view, cache.layer_view(0).struct, heads, scale, False, err, stream())
    assert err.item() == 0
    x = qkv.float().cpu().view(T, W, hd)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    t = 0
    refs = []
    for n in q_lens:
        blk = x[t:t + n]
        ref = _plain_attention(blk[:, :heads], blk[:, heads:heads + kvh], blk[:, heads + kvh:], heads, kvh, scale, window)
        got = out[t:t + n].float().cpu().view(n, heads, hd)
        assert torch.allclose(got, ref, atol=tol, rtol=tol), f"prompt of {n}"
        refs.append(blk)
        t += n
    p_far = P.softmax((x[max(0, 299 - (window - 1)) if window else 0:300, heads] @ x[299, 0]) * scale)
    assert p_far[0] > 0.5, "the far key does not dominate: the test would not see a wrong window edge"

    # one more token for each sequence, attended over the cache
    for s, n in zip(slots, q_lens):
        cache.advance(s, n)
    nxt = (torch.randn(3, W, hd, device=DEV) * 0.7).to(dtype).view(3, W * hd)
    view1, keep1 = make_batch([1, 1, 1], q_lens, slots)
    b.rope_kv_store(nxt, view1, cache.layer_view(0).struct, ident, heads, hd, b.PAIR_HALF, True, err, stream())
    out1 = torch.empty(3, heads * hd, device=DEV, dtype=dtype)
    b.attention_plain(nxt, out1, view1, cache.layer_view(0).struct, heads, scale, True, err, stream())
    assert err.item() == 0
    y = nxt.float().cpu().view(3, W, hd)
    for r, blk in enumerate(refs):
        k_all = torch.cat([blk[:, heads:heads + kvh], y[r:r + 1, heads:heads + kvh]])
        v_all = torch.cat([blk[:, heads + kvh:], y[r:r + 1, heads + kvh:]])
        ref = _plain_attention(y[r:r + 1, :heads], k_all, v_all, heads, kvh, scale, window)
        got = out1[r].float().cpu().view(1, heads, hd)
        assert torch.allclose(got, ref, atol=tol, rtol=tol), f"decode after {q_lens[r]}"
    if dtype == torch.bfloat16:
        # the split-KV kernel against its plain sibling, for several ways of splitting the keys
        for splits in (1, 3, 16):
            n = b.attention_decode_scratch_floats(3, heads, hd, splits)
            scratch = torch.full((n,), float("nan"), device=DEV)
            fast = torch.full_like(out1, float("nan"))
            assert b.attention_decode(nxt, fast, view1, cache.layer_view(0).struct, heads, scale, splits,
                                      scratch, err, stream())
            assert err.item() == 0
            assert torch.allclose(fast.float(), out1.float(), atol=tol, rtol=tol), f"split-KV, {splits} splits"


@pytest.mark.parametrize("heads,kvh,hd,window", [(32, 8, 128, 4096), (12, 2, 64, None), (3, 1, 48, 40), (8, 1, 256, None)])
def test_attention_decode_batch_with_padding(heads, kvh, hd, window):
    """A decoding batch of unequal lengths (1 to several pages), with padding sequences in
    between, against the plain kernel."""
    b = B()
    torch.manual_seed(7)
    dtype = torch.bfloat16
    cache = make_cache(kvh, hd, window, dtype, max_tokens=64 * 40, max_seq_len=1024, slots=8)
    lens = [1, 31, 32, 33, 64, 700, 437]
    slots = [cache.open_sequence() for _ in lens]
    W = heads + 2 * kvh
    scale = 1.0 / math.sqrt(hd)
    ident = torch.zeros(hd // 2, device=DEV)
    err = err_word()
    kvs = cache.layer_view(0).struct
    for s, n in zip(slots, lens):           # fill each sequence's cache with n - 1 tokens
        cache.reserve(s, n)
    cache.upload()
    filled = [n - 1 for n in lens]
    if any(filled):
        keep = [(s, n) for s, n in zip(slots, filled) if n]
        view, arrs = make_batch([n for _, n in keep], [0] * len(keep), [s for s, _ in keep])
        fill = (torch.randn(sum(filled), W * hd, device=DEV) * 0.7).to(dtype)
        b.rope_kv_store(fill, view, kvs, ident, heads, hd, b.PAIR_HALF, True, err, stream())
    # the step: 7 real sequences and 1 padding sequence (slot -1) in the middle
    order = slots[:3] + [-1] + slots[3:]
    pos0 = filled[:3] + [0] + filled[3:]
    nxt = (torch.randn(8, W, hd, device=DEV) * 0.7)
    nxt[6, :heads] *= 5.0                   # a peaked distribution for the 700-token sequence
    view1, arrs1 = make_batch([1] * 8, pos0, order)
    arrs1[2][3] = -1                         # tok_seq of the padding token
    nxt = nxt.to(dtype).view(8, W * hd)
    b.rope_kv_store(nxt, view1, kvs, ident, heads, hd, b.PAIR_HALF, True, err, stream())
    plain = torch.empty(8, heads * hd, device=DEV, dtype=dtype)
    b.attention_plain(nxt, plain, view1, kvs, heads, scale, True, err, stream())
    for splits in (1, 2, 5, 16):
        n = b.attention_decode_scratch_floats(8, heads, hd, splits)
        scratch = torch.full((n,), float("nan"), device=DEV)
        fast = torch.full_like(plain, float("nan"))
        assert b.attention_decode(nxt, fast, view1, kvs, heads, scale, splits, scratch, err, stream())
        assert err.item() == 0
        assert torch.isfinite(fast).all() and float(fast[3].abs().sum()) == 0     # padding row: zeros
        assert torch.allclose(fast.float(), plain.float(), atol=2e-2, rtol=2e-2), f"{splits} splits"
        # the tensor-core variant of the same kernel
        scratch.fill_(float("nan"))
        tc = torch.full_like(plain, float("nan"))
        assert b.attention_decode_tc(nxt, tc, view1, kvs, heads, scale, splits, scratch, err, stream())
        assert err.item() == 0
        assert torch.isfinite(tc).all() and float(tc[3].abs().sum()) == 0
        assert torch.allclose(tc.float(), plain.float(), atol=2e-2, rtol=2e-2), \
            f"tensor cores, {splits} splits: {(tc.float() - plain.float()).abs().max().item():.4g}"
        # cut by length: each sequence into as many of the `splits` parts as its share of the pages asks for
        for target in (3, 40, 1000):
            scratch.fill_(float("nan"))
            bal = torch.full_like(plain, float("nan"))
            assert b.attention_decode_tc(nxt, bal, view1, kvs, heads, scale, splits, scratch, err, stream(),
                                         target_ctas=target)
            assert err.item() == 0
            assert torch.isfinite(bal).all() and float(bal[3].abs().sum()) == 0
            assert torch.allclose(bal.float(), plain.float(), atol=2e-2, rtol=2e-2), \
                f"cut by length, {splits} parts at most, {target} CTAs aimed for"


@pytest.mark.parametrize("heads,kvh,hd", [(32, 8, 128), (12, 2, 64), (6, 3, 32)])
@pytest.mark.parametrize("window", [None, 4096])
def test_attention_decode_over_long_contexts(heads, kvh, hd, window):
    """Sequences of 9,000, 64, 4,097 and 700 tokens (over 140 pages; the window of 4,096 cuts two of
    them, one of them by a single key): the split-KV kernels with an even cut into 8 and 16 parts
    and cut by length, against the plain kernel and against a float32 statement of the same
    attention in the manner of the plain implementation.  In every sequence the last query is
    made to single out the FIRST key it may see, so that the far edge decides the result."""
    b = B()
    torch.manual_seed(11)
    dtype = torch.bfloat16
    lens = [9000, 64, 4097, 700]
    pages = sum(-(-n // 64) for n in lens)
    cache = make_cache(kvh, hd, window, dtype, max_tokens=64 * pages, max_seq_len=9024, slots=4)
    slots = [cache.open_sequence() for _ in lens]
    for s_, n in zip(slots, lens):
        cache.reserve(s_, n)
    cache.upload()
    kvs = cache.layer_view(0).struct
    W, group = heads + 2 * kvh, heads // kvh
    scale = 1.0 / math.sqrt(hd)
    ident = torch.zeros(hd // 2, device=DEV)
    err = err_word()
    fill = torch.randn(sum(n - 1 for n in lens), W, hd, device=DEV) * 0.7
    nxt = torch.randn(len(lens), W, hd, device=DEV) * 0.7
    at = 0
    for i, n in enumerate(lens):
        first = max(0, n - window) if window else 0            # the first key the token at position n - 1 sees
        nxt[i, :heads] *= 3.0
        if first < n - 1:
            fill[at + first, heads:heads + kvh] = nxt[i, 0:heads:group] * 1.0      # aligned with head 0 of each group
        at += n - 1
    fill, nxt = fill.to(dtype).view(-1, W * hd), nxt.to(dtype).view(-1, W * hd)
    view, keep = make_batch([n - 1 for n in lens], [0] * len(lens), slots)
    b.rope_kv_store(fill, view, kvs, ident, heads, hd, b.PAIR_HALF, True, err, stream())
    view1, keep1 = make_batch([1] * len(lens), [n - 1 for n in lens], slots)
    b.rope_kv_store(nxt, view1, kvs, ident, heads, hd, b.PAIR_HALF, True, err, stream())
    plain = torch.empty(len(lens), heads * hd, device=DEV, dtype=dtype)
    b.attention_plain(nxt, plain, view1, kvs, heads, scale, True, err, stream())
    assert err.item() == 0
    # the same attention stated in float32 on the bf16 values (src/layers/attention.rs:609-652)
    ref = torch.empty(len(lens), heads, hd, device=DEV)
    at, dominated = 0, 0
    f, x = fill.float().view(-1, W, hd), nxt.float().view(-1, W, hd)
    for i, n in enumerate(lens):
        k_all = torch.cat([f[at:at + n - 1, heads:heads + kvh], x[i:i + 1, heads:heads + kvh]])
        v_all = torch.cat([f[at:at + n - 1, heads + kvh:], x[i:i + 1, heads + kvh:]])
        lo = max(0, n - window) if window else 0
        for h in range(heads):
            p_ = P.softmax((k_all[lo:n, h // group] @ x[i, h]) * scale)
            ref[i, h] = p_ @ v_all[lo:n, h // group]
            if h % group == 0 and n > 64:
                dominated += int(p_[0] > 0.5)
        at += n - 1
    assert dominated >= 3 * kvh, "the first visible key does not dominate: a wrong far edge would not show"
    assert torch.allclose(plain.float().view_as(ref), ref, atol=2e-2, rtol=2e-2), "the plain kernel"
    for parts in (8, 16):
        n_s = b.attention_decode_scratch_floats(len(lens), heads, hd, parts)
        for target in (0, 64, 296, 1024):                      # 0: every sequence into all parts
            scratch = torch.full((n_s,), float("nan"), device=DEV)
            tc = torch.full_like(plain, float("nan"))
            assert b.attention_decode_tc(nxt, tc, view1, kvs, heads, scale, parts, scratch, err, stream(),
                                         target_ctas=target)
            assert err.item() == 0 and torch.isfinite(tc).all()
            what = f"{parts} parts at most, {target} CTAs aimed for"
            assert torch.allclose(tc.float(), plain.float(), atol=2e-2, rtol=2e-2), what + ": against the plain kernel"
            assert torch.allclose(tc.float().view_as(ref), ref, atol=2e-2, rtol=2e-2), what + ": against float32"
        scratch = torch.full((n_s,), float("nan"), device=DEV)
        cc = torch.full_like(plain, float("nan"))
        assert b.attention_decode(nxt, cc, view1, kvs, heads, scale, parts, scratch, err, stream())
        assert err.item() == 0
        assert torch.allclose(cc.float().view_as(ref), ref, atol=2e-2, rtol=2e-2), f"CUDA-core kernel, {parts} splits"


@pytest.mark.parametrize("heads,kvh,hd,window,pairing,rotary", [
    (32, 8, 128, None, "half", 128), (12, 2, 64, 40, "interleaved", 64), (6, 1, 32, 100, "half", 16),
    (20, 2, 48, None, "interleaved", 32)])
def test_attention_decode_with_rotation_inside(heads, kvh, hd, window, pairing, rotary):
    """The decode kernel that rotates queries and the new key and writes the cache itself, against
    the separate rotate-and-store kernel followed by the same attention kernel: same output, same
    cache afterwards; with the store switched off it reads a cache that already holds the token
    and leaves it alone.  Lengths straddle pages and (with a window) wrap the ring; groups of
    more than eight heads run as two slices."""
    b = B()
    torch.manual_seed(11)
    dtype = torch.bfloat16
    W = heads + 2 * kvh
    scale = 1.0 / math.sqrt(hd)
    code = b.PAIR_HALF if pairing == "half" else b.PAIR_INTERLEAVED
    inv_freq = (10000.0 ** (-torch.arange(rotary // 2, dtype=torch.float64) * 2 / rotary)).float().to(DEV)
    lens = [1, 64, 65, 300, 129]
    fill = (torch.randn(sum(n - 1 for n in lens), W * hd, device=DEV) * 0.7).to(dtype)
    nxt = (torch.randn(len(lens) + 1, W * hd, device=DEV) * 0.7).to(dtype)
    err = err_word()
    caches, views = [], []
    for _ in range(2):                        # two caches with the same history
        cache = make_cache(kvh, hd, window, dtype, max_tokens=64 * 24, max_seq_len=512, slots=6)
        slots = [cache.open_sequence() for _ in lens]
        for s_, n in zip(slots, lens):
            cache.reserve(s_, n)
        cache.upload()
        keep = [(s_, n - 1) for s_, n in zip(slots, lens) if n > 1]
        view, arrs = make_batch([n for _, n in keep], [0] * len(keep), [s_ for s_, _ in keep])
        b.rope_kv_store(fill.clone(), view, cache.layer_view(0).struct, inv_freq, heads, rotary, code, True, err, stream())
        caches.append(cache)
        views.append(cache.layer_view(0))
    order = slots[:2] + [-1] + slots[2:]      # a padding sequence in the middle
    pos0 = [lens[0] - 1, lens[1] - 1, 0] + [n - 1 for n in lens[2:]]
    step, arrs1 = make_batch([1] * 6, pos0, order)
    arrs1[2][2] = -1
    for splits in (1, 3, 8):
        n = b.attention_decode_scratch_floats(6, heads, hd, splits)
        scratch = torch.full((n,), float("nan"), device=DEV)
        # separately: rotate and store, then attend
        rotated = nxt.clone()
        b.rope_kv_store(rotated, step, views[0].struct, inv_freq, heads, rotary, code, True, err, stream())
        want = torch.full((6, heads * hd), float("nan"), device=DEV, dtype=dtype)
        assert b.attention_decode_tc(rotated, want, step, views[0].struct, heads, scale, splits, scratch, err, stream())
        # in one kernel, from the raw projection, into the second cache
        raw = nxt.clone()
        got = torch.full_like(want, float("nan"))
        scratch.fill_(float("nan"))
        assert b.attention_decode_tc_rope(raw, got, step, views[1].struct, heads, scale, splits, scratch, inv_freq,
                                          rotary, code, True, err, stream())
        assert err.item() == 0
        assert torch.equal(raw, nxt), "the fused kernel must leave the projection as it is"
        assert torch.isfinite(got).all() and float(got[2].abs().sum()) == 0
        diff = (got.float() - want.float()).abs().max().item()
        assert diff <= 1e-2, f"{splits} splits: output differs by {diff:.4g}"
        live = sorted(set(p_ for s_ in slots for p_ in caches[0].kv_groups[0].pages_of(s_)))
        for a_, b_ in ((views[0].k, views[1].k), (views[0].v, views[1].v)):
            ka, kb = a_[live].float(), b_[live].float()
            both = torch.isfinite(ka) & torch.isfinite(kb)
            assert torch.equal(torch.isfinite(ka), torch.isfinite(kb)), "different rows were written"
            assert (ka[both] - kb[both]).abs().max().item() <= 2.0 ** -6, "the caches differ"
        # store off: the second cache holds the token already; output as before, cache untouched
        before = (views[1].k.clone(), views[1].v.clone())
        again = torch.full_like(want, float("nan"))
        scratch.fill_(float("nan"))
        assert b.attention_decode_tc_rope(raw, again, step, views[1].struct, heads, scale, splits, scratch, inv_freq,
                                          rotary, code, False, err, stream())
        assert err.item() == 0
        assert (again.float() - want.float()).abs().max().item() <= 1e-2
        assert torch.equal(before[0].view(torch.int16), views[1].k.view(torch.int16))
        assert torch.equal(before[1].view(torch.int16), views[1].v.view(torch.int16))


def test_sampling_greedy_and_errors():
    b = B()
    logits = torch.randn(5, 1000, device=DEV)
    logits[1, 7] = logits[1, 900] = 50.0            # a tie: the first index wins
    logits[2, 999] = 60.0
    logits[3, 0] = 60.0
    out = torch.empty(5, dtype=torch.int32, device=DEV)
    err = err_word()
    b.sample_greedy(logits, out, err, stream())
    assert out.tolist() == [int(logits[0].argmax()), 7, 999, 0, int(logits[4].argmax())] and err.item() == 0
    for r in range(5):
        assert out[r].item() == P.sample_greedy(logits[r].tolist())
    logits[4, 3] = float("nan")
    b.sample_greedy(logits, out, err, stream())
    assert err.item() == b.ERR_NONFINITE_LOGIT


@pytest.mark.parametrize("vocab", [331, 32000, 1024])
@pytest.mark.parametrize("temperature", [0.7, 1.0, 2.5])
def test_sampling_temperature_follows_the_cdf(vocab, temperature):
    b = B()
    torch.manual_seed(6)
    rows = 64
    logits = torch.randn(rows, vocab, device=DEV) * 3
    req = torch.arange(rows, dtype=torch.int32, device=DEV) * 3 + 1
    step = torch.full((rows,), 9, dtype=torch.int32, device=DEV)
    seed = 0x1234_5678_9ABC_DEF0
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    draws = torch.empty(rows, device=DEV)
    err = err_word()
    b.sample_temperature(logits, temperature, seed, req, step, out, err, stream())
    b.uniform_draws(seed, req, step, draws, stream())
    assert err.item() == 0
    for r in range(rows):
        u = P.uniform_draw(seed, int(req[r]), 9)
        assert abs(draws[r].item() - u) < 1e-9
        cdf = P.temperature_cdf(logits[r].cpu(), temperature)
        i = int(out[r])
        lo = float(cdf[i - 1]) if i > 0 else 0.0
        assert lo - 1e-5 <= u <= float(cdf[i]) + 1e-5, (r, i, u, lo, float(cdf[i]))
    # the same request and step give the same token whatever else is in the batch
    out2 = torch.empty(3, dtype=torch.int32, device=DEV)
    pick = [40, 2, 17]
    b.sample_temperature(logits[pick].contiguous(), temperature, seed, req[pick].contiguous(),
                         step[pick].contiguous(), out2, err, stream())
    assert out2.tolist() == out[pick].tolist()
    # a distribution with all its mass on one id
    peaked = torch.full((1, vocab), -50.0, device=DEV)
    peaked[0, vocab - 1] = 50.0
    b.sample_temperature(peaked, temperature, seed, req[:1], step[:1], out2[:1], err, stream())
    assert out2[0].item() == vocab - 1


@pytest.mark.parametrize("heads,kvh,hd,window", [(4, 2, 16, 16), (6, 1, 32, None), (3, 3, 48, 70), (8, 2, 128, None),
                                                 (4, 4, 128, 100), (5, 5, 80, 33), (2, 1, 256, 130), (6, 2, 64, None),
                                                 (3, 1, 64, 200), (2, 2, 128, 129)])
def test_attention_prefill_against_plain_kernel(heads, kvh, hd, window):
    """The tensor-core prompt attention against its plain sibling: unequal prompts (a single
    token, lengths around the 64-wide tiles, several tiles), windows that cut tiles at odd
    places, and one far key that carries the output of the last query."""
    b = B()
    torch.manual_seed(8)
    dtype = torch.bfloat16
    q_lens = [1, 63, 64, 65, 300, 129]
    T, Wd = sum(q_lens), heads + 2 * kvh
    scale = 1.0 / math.sqrt(hd)
    cache = make_cache(kvh, hd, window, dtype)          # only its geometry is used
    view, keep = make_batch(q_lens, [0] * len(q_lens), list(range(len(q_lens))))
    qkv = torch.randn(T, Wd, hd, device=DEV) * 0.7
    last = sum(q_lens[:5]) - 1                           # last query of the 300-token prompt
    far = last - (window - 1) if window else last - 299
    qkv[last, :heads] *= 4.0
    qkv[far, heads:heads + kvh] = qkv[last, 0:heads:heads // kvh]
    qkv = qkv.to(dtype).view(T, Wd * hd)
    err = err_word()
    plain = torch.empty(T, heads * hd, device=DEV, dtype=dtype)
    b.attention_plain(qkv, plain, view, cache.layer_view(0).struct, heads, scale, False, err, stream())
    for legacy in (True, False):        # the mma.sync kernel; then tcgen05 where the head size has it
        fast = torch.full_like(plain, float("nan"))
        assert b.attention_prefill(qkv, fast, view, heads, kvh, hd, window or 0, scale, max(q_lens), stream(),
                                   err=err, legacy=legacy)
        torch.cuda.synchronize()
        assert err.item() == 0, b.describe_error_bits(err.item())
        assert torch.isfinite(fast).all()
        assert torch.allclose(fast.float(), plain.float(), atol=2e-2, rtol=2e-2), \
            f"legacy={legacy}: max diff {(fast.float() - plain.float()).abs().max().item():.4g}"
    x = qkv.float().cpu().view(T, Wd, hd)
    lo = far
    p_far = P.softmax((x[lo:last + 1, heads] @ x[last, 0]) * scale)
    assert p_far[0] > 0.5, "the far key does not dominate"
    # the kernel the engine runs for this head size, also against the per-row statement of the
    # same attention (softmax of the plain implementation), not only against its sibling kernel
    t = 0
    for n in q_lens:
        blk = x[t:t + n]
        ref = _plain_attention(blk[:, :heads], blk[:, heads:heads + kvh], blk[:, heads + kvh:], heads, kvh, scale, window)
        got = fast[t:t + n].float().cpu().view(n, heads, hd)
        assert torch.allclose(got, ref, atol=2e-2, rtol=2e-2), f"prompt of {n} tokens against the per-row statement"
        t += n
