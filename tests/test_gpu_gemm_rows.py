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
