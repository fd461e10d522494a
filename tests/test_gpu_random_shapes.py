"""The projections at shapes drawn at random, through the dispatch the parts use (`Linear.apply`, the gated
form of the feed-forward): token counts from one to several tiles, widths and depths that are multiples of 8
but of nothing larger, layer-sized and tiny.  Against the float64 product of the same bfloat16 operands.
Whichever kernel the dispatch picks (rows kernel, tcgen05 with or without split-K, gated, or the plain
kernel for what they refuse), the result is the product."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
N_CASES = int(os.environ.get("IERT_TEST_RANDOM_SHAPES", "24"))     # (more for a longer hunt)


def draw(rng):
    M = int(rng.choice([1, 2, 7, 8, 9, 16, 17, 31, 33, 64, 65, 100, 128, 130, 257, 300, 513, 700]))
    N = int(rng.choice([8, 24, 104, 128, 136, 520, 1000, 1536, 2048, 4096, 6144])) + 8 * int(rng.integers(0, 3))
    K = int(rng.choice([8, 40, 64, 72, 200, 512, 1096, 2048, 4096, 5120])) + 8 * int(rng.integers(0, 3))
    return M, N, K


CASES = [draw(np.random.default_rng(500 + i)) for i in range(N_CASES)]


def _rt():
    from inference_engine_rust_b200.parts import Runtime
    return Runtime(torch.bfloat16, DEV)


def _check(out, ref, K, what):
    scale = (K ** 0.5) * 0.5
    bound = 2e-3 * scale + (2.0 ** -8) * ref.abs() * (out.dtype == torch.bfloat16)
    diff = (out.double() - ref).abs()
    assert torch.isfinite(out).all() and bool((diff <= bound).all()), f"{what}: max diff {diff.max().item():.4g}"


@pytest.mark.parametrize("M,N,K", CASES)
def test_projection_at_a_random_shape(M, N, K):
    from inference_engine_rust_b200.csrc import bindings as B
    from inference_engine_rust_b200.parts import Linear
    rt = _rt()
    g = torch.Generator(device=DEV).manual_seed(M * 1000003 + N * 1009 + K)
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.5).bfloat16()
    lin = Linear(w, rt)
    ref = x.double() @ w.double().t()
    out = torch.full((M, N), float("nan"), device=DEV, dtype=torch.bfloat16)
    lin.apply(x, out, M, B.stream_ptr())
    res0 = torch.randn(M, N, device=DEV, generator=g)
    res = res0.clone()
    lin.apply(x, res, M, B.stream_ptr(), add_residual=True)
    torch.cuda.synchronize()
    assert rt.err.item() == 0, B.describe_error_bits(rt.err.item())
    _check(out, ref, K, f"store M={M} N={N} K={K}")
    _check(res, ref + res0.double(), K, f"residual add M={M} N={N} K={K}")


@pytest.mark.parametrize("M,N,K", CASES[:max(12, N_CASES // 2)])
def test_gated_projection_at_a_random_shape(M, N, K):
    """silu(x . Wg^T) * (x . Wu^T) through the feed-forward's own dispatch (one gated kernel where it is taken,
    else the product and the activation kernel)."""
    from inference_engine_rust_b200.config.specs import PartSpec
    from inference_engine_rust_b200.csrc import bindings as B
    from inference_engine_rust_b200.parts import part_class
    from inference_engine_rust_b200.parts.base import StepContext
    rt = _rt()
    inter = N
    g = torch.Generator(device=DEV).manual_seed(M * 7919 + N * 31 + K)
    ffn = part_class("ffn", "swiglu")(PartSpec("swiglu", {"hidden_size": K, "intermediate_size": inter}), rt)
    wg = (torch.randn(inter, K, device=DEV, generator=g) * 0.3).bfloat16()
    wu = (torch.randn(inter, K, device=DEV, generator=g) * 0.3).bfloat16()
    wd = (torch.randn(K, inter, device=DEV, generator=g) * 0.1).bfloat16()
    ffn.load({"gate_proj.weight": wg, "up_proj.weight": wu, "down_proj.weight": wd})
    x = (torch.randn(M, K, device=DEV, generator=g) * 0.5).bfloat16()
    res0 = torch.randn(M, K, device=DEV, generator=g)
    res = res0.clone()
    ctx = StepContext(kind="prompt", batch=None, n_tokens=M, n_seqs=1, q_lens=[M], pos0=[0], slots=[0],
                      stream=B.stream_ptr(), rt=rt)
    ffn.forward(x, res, ctx)
    torch.cuda.synchronize()
    assert rt.err.item() == 0, B.describe_error_bits(rt.err.item())
    gate, up = x.double() @ wg.double().t(), x.double() @ wu.double().t()
    act = (gate * torch.sigmoid(gate) * up).to(torch.bfloat16).double()      # the activation is stored in bfloat16
    ref = res0.double() + act @ wd.double().t()
    # one bfloat16 rounding of each activation value, carried through the down projection
    bound = 2e-3 * (K ** 0.5) + 2.0 ** -7 * (act.abs() @ wd.double().abs().t())
    diff = (res.double() - ref).abs()
    assert torch.isfinite(res).all() and bool((diff <= bound).all()), f"M={M} I={inter} H={K}: max diff {diff.max().item():.4g}"
