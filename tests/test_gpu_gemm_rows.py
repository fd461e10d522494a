"""The projection kernel of one-token steps that gives every CTA 16 weight rows over all of k (no
split-K), alone, against a float64 product of the same bf16 operands: every token group (up to
8, 16, 32 tokens), widths and k that are no multiple of the tiles, rings shorter and longer than
the k loop, both output types and the residual add; repeatable to the bit."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def run(M, N, K, mode, out_dtype, **force):
    from inference_engine_rust_b200.csrc import bindings as B
    g = torch.Generator(device=DEV).manual_seed(M * 1000003 + N * 1009 + K)
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.5).bfloat16()
    ref = x.double() @ w.double().t()
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    if mode == B.GEMM_ADD_RESIDUAL:
        out = torch.randn(M, N, device=DEV, generator=g)
        ref = ref + out.double()
    else:
        out = torch.full((M, N), float("nan"), device=DEV, dtype=out_dtype)
    assert B.gemm_rows(x, w, out, M, mode, err, B.stream_ptr(), **force), "the kernel refused operands it should take"
    torch.cuda.synchronize()
    assert err.item() == 0, B.describe_error_bits(err.item())
    bound = 2e-3 * (K ** 0.5) * 0.5 + (2.0 ** -8) * ref.abs() * (out.dtype == torch.bfloat16)
    diff = (out.double() - ref).abs()
    assert torch.isfinite(out).all() and bool((diff <= bound).all()), \
        f"M={M} N={N} K={K} {force}: max diff {diff.max().item():.4g}"
    return out


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16, 17, 32])
@pytest.mark.parametrize("N,K", [(4096, 4096), (331, 520), (16, 64), (100, 88), (6144, 1024), (4096, 14336)])
def test_shapes(M, N, K):
    from inference_engine_rust_b200.csrc import bindings as B
    run(M, N, K, B.GEMM_STORE, torch.bfloat16)
    run(M, N, K, B.GEMM_STORE, torch.float32)
    a = run(M, N, K, B.GEMM_ADD_RESIDUAL, torch.float32)
    b = run(M, N, K, B.GEMM_ADD_RESIDUAL, torch.float32)
    assert torch.equal(a, b), "two identical runs differ"


@pytest.mark.parametrize("stages", [1, 2, 3, 9])
def test_rings_shorter_and_longer_than_the_k_loop(stages):
    from inference_engine_rust_b200.csrc import bindings as B
    run(8, 256, 4096, B.GEMM_STORE, torch.float32, force_stages=stages)     # 8 uses of the ring
    run(8, 256, 4104, B.GEMM_STORE, torch.float32, force_stages=stages)     # k no multiple of 64: a copy per k-block
    run(20 if stages < 4 else 5, 48, 200, B.GEMM_ADD_RESIDUAL, torch.float32, force_stages=stages)   # a single, partly empty use


def test_refuses_what_it_does_not_take():
    from inference_engine_rust_b200.csrc import bindings as B
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    w = torch.randn(64, 128, device=DEV).bfloat16()
    out = torch.zeros(33, 64, device=DEV)
    assert B.gemm_rows(torch.randn(33, 128, device=DEV).bfloat16(), w, out, 33, B.GEMM_STORE, err, B.stream_ptr()) is False
    w100 = torch.randn(64, 100, device=DEV).bfloat16()
    assert B.gemm_rows(torch.randn(4, 100, device=DEV).bfloat16(), w100, out, 4, B.GEMM_STORE, err, B.stream_ptr()) is False
    assert float(out.abs().sum()) == 0


def test_a_token_does_not_depend_on_the_others():
    """Row t of the result is the same to the bit whether the step holds 1, 8 or 32 tokens: the
    order of the additions depends on k alone."""
    from inference_engine_rust_b200.csrc import bindings as B
    g = torch.Generator(device=DEV).manual_seed(1)
    x = torch.randn(32, 1024, device=DEV, generator=g).bfloat16()
    w = torch.randn(768, 1024, device=DEV, generator=g).bfloat16()
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    rows = []
    for M in (1, 8, 32):
        out = torch.empty(M, 768, device=DEV)
        assert B.gemm_rows(x, w, out, M, B.GEMM_STORE, err, B.stream_ptr())
        rows.append(out[0].clone())
    assert torch.equal(rows[0], rows[1]) and torch.equal(rows[0], rows[2])


# ---- an RMSNorm split in two around the kernel boundary ------------------------------------------


def _parts_of(rows, parts):
    """Partial sums of squares of each row over `parts` runs of columns (float64 -> float32)."""
    M, H = rows.shape
    per = -(-H // parts)
    pad = torch.zeros(M, per * parts, device=rows.device, dtype=torch.float64)
    pad[:, :H] = rows.double()
    return (pad.view(M, parts, per) ** 2).sum(-1).float().contiguous()


@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (8, 6144, 4096), (13, 331, 520), (16, 64, 64)])
@pytest.mark.parametrize("wdt", [torch.bfloat16, torch.float32])
def test_residual_add_writes_the_next_norms_first_half(M, N, K, wdt):
    """Beside the new residual rows: bf16(row * weight) and one partial sum of squares per CTA, which
    add up to the rows' sums of squares; everything repeatable to the bit."""
    from inference_engine_rust_b200.csrc import bindings as B
    g = torch.Generator(device=DEV).manual_seed(M + N + K)
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.5).bfloat16()
    nw = (1.0 + 0.1 * torch.randn(N, device=DEV, generator=g)).to(wdt)
    res0 = torch.randn(M, N, device=DEV, generator=g)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    outs = []
    for _ in range(2):
        out = res0.clone()
        scaled = torch.full((M, N), float("nan"), device=DEV, dtype=torch.bfloat16)
        sumsq = torch.full((M, -(-N // 16)), float("nan"), device=DEV)
        ahead = B.norm_ahead(nw, scaled, sumsq)
        assert B.gemm_rows(x, w, out, M, B.GEMM_ADD_RESIDUAL, err, B.stream_ptr(), ahead=ahead)
        torch.cuda.synchronize()
        assert err.item() == 0 and ahead.parts == -(-N // 16)
        ref = x.double() @ w.double().t() + res0.double()
        assert bool(((out.double() - ref).abs() <= 2e-3 * (K ** 0.5) * 0.5).all())
        assert torch.equal(scaled, (out * nw.float()).bfloat16()), "scaled = bf16(new row * weight)"
        assert torch.allclose(sumsq.double().sum(-1), (out.double() ** 2).sum(-1), rtol=1e-5)
        assert torch.allclose(sumsq, _parts_of(out, ahead.parts), rtol=1e-4, atol=1e-6) or N % 16
        outs.append((out, scaled, sumsq))
    assert all(torch.equal(a, b) for a, b in zip(*outs))


@pytest.mark.parametrize("M,N,K,parts", [(1, 6144, 4096, 256), (8, 6144, 4096, 256), (16, 200, 520, 1), (5, 64, 64, 4), (8, 4096, 4096, 33)])
def test_projection_applies_the_norms_second_half(M, N, K, parts):
    """x = bf16(rows * weight) with the rows' partial sums of squares: the projection multiplies its
    outputs by each row's 1 / sqrt(mean + eps); against the whole norm followed by the product."""
    from inference_engine_rust_b200.csrc import bindings as B
    g = torch.Generator(device=DEV).manual_seed(M * 3 + N + K + parts)
    rows = torch.randn(M, K, device=DEV, generator=g) * 3.0
    nw = 1.0 + 0.1 * torch.randn(K, device=DEV, generator=g)
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.5).bfloat16()
    eps = 1e-5
    scaled = (rows * nw).bfloat16()
    sumsq = _parts_of(rows, parts)
    rstd = 1.0 / torch.sqrt((rows.double() ** 2).mean(-1, keepdim=True) + eps)
    ref = (scaled.double() * rstd) @ w.double().t()          # the rounded first half, the factor in full precision
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.full((M, N), float("nan"), device=DEV)
    scale = B.RowScale(sumsq=sumsq.data_ptr(), parts=parts, hidden=K, eps=eps)
    assert B.gemm_rows(scaled, w, out, M, B.GEMM_STORE, err, B.stream_ptr(), scale=scale)
    torch.cuda.synchronize()
    assert err.item() == 0
    bound = 2e-3 * (K ** 0.5) * 0.5 + 1e-5 * ref.abs()
    diff = (out.double() - ref).abs()
    assert torch.isfinite(out).all() and bool((diff <= bound).all()), f"max diff {diff.max().item():.4g}"


@pytest.mark.parametrize("M,I,K,parts", [(1, 14336, 4096, 256), (8, 14336, 4096, 256), (16, 9600, 520, 1), (40, 14336, 256, 16)])
def test_gated_product_applies_the_norms_second_half(M, I, K, parts):
    from inference_engine_rust_b200.csrc import bindings as B
    g = torch.Generator(device=DEV).manual_seed(M + I + K)
    rows = torch.randn(M, K, device=DEV, generator=g) * 2.0
    nw = 1.0 + 0.1 * torch.randn(K, device=DEV, generator=g)
    w = (torch.randn(2 * I, K, device=DEV, generator=g) * (2.0 / K ** 0.5)).bfloat16()
    eps = 1e-6
    scaled = (rows * nw).bfloat16()
    sumsq = _parts_of(rows, parts)
    rstd = 1.0 / torch.sqrt((rows.double() ** 2).mean(-1, keepdim=True) + eps)
    xn = scaled.double() * rstd
    gate, up = xn @ w[:I].double().t(), xn @ w[I:].double().t()
    ref = gate * torch.sigmoid(gate) * up
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    act = torch.full((M, I), float("nan"), device=DEV, dtype=torch.bfloat16)
    scale = B.RowScale(sumsq=sumsq.data_ptr(), parts=parts, hidden=K, eps=eps)
    assert B.gemm_tc_gated_scaled(scaled, w, act, M, scale, err, B.stream_ptr())
    torch.cuda.synchronize()
    assert err.item() == 0
    diff = (act.double() - ref).abs()
    bound = 1e-3 + (2.0 ** -8) * ref.abs() + 1e-3 * (gate.abs() + 1) * up.abs()
    assert torch.isfinite(act).all() and bool((diff <= bound).all()), f"max diff {diff.max().item():.4g}"


@pytest.mark.parametrize("tdt,wdt", [(torch.bfloat16, torch.bfloat16), (torch.float32, torch.float32)])
def test_embedding_writes_the_first_norms_first_half(tdt, wdt):
    from inference_engine_rust_b200.csrc import bindings as B
    torch.manual_seed(3)
    table = torch.randn(331, 1000, device=DEV).to(tdt)
    nw = (1.0 + 0.1 * torch.randn(1000, device=DEV)).to(wdt)
    ids = torch.tensor([5, 330, 0, 17, 5], dtype=torch.int32, device=DEV)
    x = torch.empty(5, 1000, device=DEV)
    scaled = torch.empty(5, 1000, device=DEV, dtype=torch.bfloat16)
    sumsq = torch.empty(5, 1, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    ahead = B.norm_ahead(nw, scaled, sumsq)
    assert B.embed_gather(table, ids, x, 1.5, err, B.stream_ptr(), ahead=ahead) == 1
    torch.cuda.synchronize()
    want = table[ids.long()].float() * 1.5
    assert torch.equal(x, want) and torch.equal(scaled, (want * nw.float()).bfloat16())
    assert torch.allclose(sumsq[:, 0].double(), (want.double() ** 2).sum(-1), rtol=1e-5)
