"""The plain implementation against the numeric vectors of the reference's own unit tests,
and against itself where a formula has two statements."""
import math

import pytest
import torch

from plain import mistral_plain as P


def test_rmsnorm_reference_vector():
    # src/ops/rmsnorm.rs:66-78
    out = P.rmsnorm(torch.tensor([[0.5, 1.0, 1.5]]), torch.tensor([0.2, 0.3, 0.4]), 1e-6)
    assert torch.allclose(out, torch.tensor([[0.092582, 0.277746, 0.555492]]), atol=1e-5)


def test_rope_reference_vectors():
    # src/ops/rope.rs:63-77: base 1, pos 1, one pair; and position 0 is the identity
    v = P.rope(torch.tensor([1.0, 2.0]), 1.0, 1, 2, 2, "interleaved")
    assert torch.allclose(v, torch.tensor([-1.1426396, 1.9220756]), atol=1e-5)
    v = P.rope(torch.tensor([1.0, 0.0, 1.0, 0.0]), 10000.0, 0, 4, 4, "interleaved")
    assert torch.allclose(v, torch.tensor([1.0, 0.0, 1.0, 0.0]), atol=1e-6)


def test_rope_pairings_are_one_rotation_under_a_permutation():
    # rotating (2k, 2k+1) of a permuted head equals rotating (k, k+half) of the head itself
    torch.manual_seed(0)
    hd = 16
    v = torch.randn(hd)
    perm = torch.cat([torch.arange(0, hd, 2), torch.arange(1, hd, 2)])   # interleaved -> half order
    a = P.rope(v, 10000.0, 7, hd, hd, "interleaved")[perm]
    b = P.rope(v[perm], 10000.0, 7, hd, hd, "half")
    assert torch.allclose(a, b, atol=1e-6)


def test_rope_partial_rotary_passes_through():
    v = torch.arange(8, dtype=torch.float32)
    out = P.rope(v, 100.0, 3, 8, 4, "half")
    assert torch.equal(out[4:], v[4:]) and not torch.allclose(out[:4], v[:4])


def test_softmax_reference_vector():
    # src/ops/softmax.rs:35-48
    out = P.softmax(torch.tensor([0.0, 1.0]))
    assert torch.allclose(out, torch.tensor([0.2689414, 0.7310586]), atol=1e-6)
    assert abs(out.sum().item() - 1) < 1e-6


def test_swiglu_reference_vector():
    # src/ops/swiglu.rs:40-50
    out = P.swiglu(torch.tensor([0.0, 1.0]), torch.tensor([1.0, 1.0]))
    assert torch.allclose(out, torch.tensor([0.0, 0.7310586]), atol=1e-6)
    big = P.sigmoid(torch.tensor([-200.0, 200.0]))
    assert torch.isfinite(big).all() and big[0] == 0 and big[1] == 1


def test_matmul_layout_reference_vector():
    # src/ops/matmul.rs:454-464: x = [1, 2], weight buffer [1, 2, 3, 4] as rows [1,2], [3,4]
    out = P.matmul(torch.tensor([[1.0, 2.0]]), torch.tensor([[1.0, 2.0], [3.0, 4.0]]))
    assert torch.equal(out, torch.tensor([[5.0, 11.0]]))


def test_sampling_reference_vectors():
    # src/engine/sampling.rs:86-115
    assert P.sample_greedy([0.0, 2.0, 1.0]) == 1
    assert P.sample_greedy([1.0, 3.0, 3.0]) == 1          # first of the tie
    with pytest.raises(ValueError):
        P.sample_greedy([])
    with pytest.raises(ValueError):
        P.sample_greedy([0.0, float("nan")])
    for t in (0.0, -1.0, float("inf")):
        with pytest.raises(ValueError):
            P.sample_temperature(torch.tensor([1.0, 2.0]), t, 0.5)
    logits = torch.tensor([0.0, 1.0, 0.0])
    cdf = P.temperature_cdf(logits, 1.0)
    assert P.sample_temperature(logits, 1.0, 0.0) == 0
    assert P.sample_temperature(logits, 1.0, float(cdf[0]) + 1e-9) == 1
    assert P.sample_temperature(logits, 1.0, 0.999999) == 2


def test_philox_known_answer():
    # Random123 known-answer vectors for philox4x32-10
    assert P.philox4x32_10([0, 0, 0, 0], [0, 0]) == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
    assert P.philox4x32_10([0xffffffff] * 4, [0xffffffff] * 2) == [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]
    assert P.philox4x32_10([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], [0xa4093822, 0x299f31d0]) == \
        [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]
    r = P.uniform_draw(7, 3, 5)
    assert 0.0 <= r < 1.0 and r == P.uniform_draw(7, 3, 5) and r != P.uniform_draw(7, 3, 6)


def test_attention_window_and_causality():
    # a key outside the window or in the future must not change the output
    torch.manual_seed(1)
    H, heads, kvh, hd, T, W = 32, 4, 2, 8, 12, 5
    xn = torch.randn(T, H)
    wq, wk, wv, wo = (torch.randn(heads * hd, H) * .2, torch.randn(kvh * hd, H) * .2,
                      torch.randn(kvh * hd, H) * .2, torch.randn(H, heads * hd) * .2)
    kw = dict(heads=heads, kv_heads=kvh, head_dim=hd, rope_theta=1e4, window=W)
    y = P.attention_layer(xn, wq, wk, wv, wo, **kw)
    xn2 = xn.clone()
    xn2[0] += 5.0                                    # position 0 is outside the window of rows >= 5
    y2 = P.attention_layer(xn2, wq, wk, wv, wo, **kw)
    assert torch.allclose(y[W:], y2[W:], atol=1e-6) and not torch.allclose(y[:W], y2[:W], atol=1e-3)
    xn3 = xn.clone()
    xn3[-1] += 5.0                                   # the last row is in nobody else's past
    y3 = P.attention_layer(xn3, wq, wk, wv, wo, **kw)
    assert torch.allclose(y[:-1], y3[:-1], atol=1e-6)


def test_forward_prefix_consistency():
    # logits of a prefix do not depend on what follows (no cache here: whole sequences)
    from helpers import TINY_A
    from inference_engine_rust_b200 import Model, config_from_dict, spec_of
    from inference_engine_rust_b200.parts.base import Runtime
    from inference_engine_rust_b200.weights import RandomSource
    cfg = dict(TINY_A)
    m = Model(spec_of(config_from_dict(cfg)), Runtime(dtype=torch.float32, device="cpu"))
    src = RandomSource(m.expected_tensors(), 3, 0.1, dtype=torch.float32)
    w = {n: src.get(n) for n in src.names()}
    ids = list(range(5, 45))
    full = P.forward(cfg, w, ids)
    part = P.forward(cfg, w, ids[:17])
    assert torch.allclose(full[:17], part, atol=1e-5)
    assert full.shape == (40, cfg["vocab_size"])
    gen = P.generate_greedy(cfg, w, ids[:6], 4)
    assert len(gen) == 4 and gen[0] == P.sample_greedy(P.forward(cfg, w, ids[:6])[-1].tolist())


def test_plain_implementation_against_its_committed_outputs():
    """The plain implementation still computes what it computed when tests/golden was written
    (its own earlier output, not the reference's: see tests/golden/make_golden.py)."""
    import importlib.util
    import os
    import numpy as np
    here = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(here, "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    want = np.load(os.path.join(here, "plain_tiny_logits.npz"))
    got = mod.compute()
    assert sorted(want.files) == sorted(got)
    for k in want.files:
        if k.endswith("_ids"):
            assert np.array_equal(want[k], got[k]), k
        else:
            assert np.allclose(want[k], got[k], atol=1e-5, rtol=1e-5), f"{k}: max diff {np.abs(want[k] - got[k]).max()}"
