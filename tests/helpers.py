"""Shared by the tests: the tiny configurations (differing in every size and option),
random model folders in temporary directories, weights for the plain implementation, and
the comparison used for logits."""
from __future__ import annotations

import os
from typing import Dict, List, Sequence

import numpy as np
import torch

# Tiny A: 2 layers, hidden 64, 4 heads / 2 kv heads (grouped), head_dim 16 (heads*head_dim =
# hidden), intermediate 192, vocab 256, theta 1e4, window 16, eps 1e-5.
TINY_A = {
    "architectures": ["MistralForCausalLM"], "model_type": "mistral",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 192, "vocab_size": 256, "rope_theta": 10000.0,
    "sliding_window": 16, "rms_norm_eps": 1e-5, "max_position_embeddings": 512,
    "tie_word_embeddings": False, "hidden_act": "silu", "bos_token_id": 1, "eos_token_id": 2,
}
# Tiny B: 3 layers, hidden 96, 6 heads / 1 kv head (multi-query), head_dim 32 (heads*head_dim =
# 192 != hidden), intermediate 160, vocab 384 (no power of two), theta 1e6, no window, eps 1e-6.
TINY_B = {
    "architectures": ["MistralForCausalLM"], "model_type": "mistral",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 6, "num_key_value_heads": 1,
    "head_dim": 32, "intermediate_size": 160, "vocab_size": 384, "rope_theta": 1000000.0,
    "sliding_window": None, "rms_norm_eps": 1e-6, "max_position_embeddings": 1024,
    "tie_word_embeddings": False, "hidden_act": "silu", "bos_token_id": 1, "eos_token_id": 2,
}
# Tiny C: odd sizes everywhere (hidden and vocabulary no multiple of 8, head_dim 48, tied output).
TINY_C = {
    "architectures": ["MistralForCausalLM"], "model_type": "mistral",
    "num_hidden_layers": 2, "hidden_size": 88, "num_attention_heads": 3, "num_key_value_heads": 3,
    "head_dim": 48, "intermediate_size": 200, "vocab_size": 331, "rope_theta": 50000.0,
    "sliding_window": 70, "rms_norm_eps": 1e-5, "max_position_embeddings": 512,
    "tie_word_embeddings": True, "hidden_act": "silu", "bos_token_id": 1, "eos_token_id": 2,
}
# Tiny D: sizes the tensor-core kernels do not take (widths that are no multiple of 8, head_dim
# 24): every product and the attention fall back to the plain kernels, also in bfloat16.
TINY_D = {
    "architectures": ["MistralForCausalLM"], "model_type": "mistral",
    "num_hidden_layers": 2, "hidden_size": 100, "num_attention_heads": 5, "num_key_value_heads": 1,
    "head_dim": 24, "intermediate_size": 76, "vocab_size": 130, "rope_theta": 10000.0,
    "sliding_window": 40, "rms_norm_eps": 1e-5, "max_position_embeddings": 512,
    "tie_word_embeddings": False, "hidden_act": "silu", "bos_token_id": 1, "eos_token_id": 2,
}
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D}

WEIGHT_STD = 0.1      # larger than the customary 0.02 so that attention is not uniform


def make_folder(tmp_path, cfg: dict, seed: int = 0, dtype: str = "float32", std: float = WEIGHT_STD) -> str:
    from inference_engine_rust_b200 import write_random_model
    d = os.path.join(str(tmp_path), f"model_{abs(hash((str(sorted(cfg.items())), seed, dtype, std))) % 10**8}")
    if not os.path.isdir(d):
        write_random_model(d, dict(cfg), seed=seed, dtype=dtype, std=std)
    return d


def plain_weights(model_dir: str) -> Dict[str, torch.Tensor]:
    """Read a folder's tensors with the `safetensors` package (not the package under test)
    and widen them to float32."""
    from safetensors.torch import load_file
    return {k: v.to(torch.float32) for k, v in load_file(os.path.join(model_dir, "model.safetensors")).items()}


def prompts_for(cfg: dict, lengths: Sequence[int], seed: int = 0) -> List[List[int]]:
    g = np.random.default_rng(seed)
    return [g.integers(0, cfg["vocab_size"], size=n).tolist() for n in lengths]


# Tolerances for logits.
#   float32: the engine and the plain implementation differ by summation order, by the
#   exp / sin / cos implementations and by how the rotary angle is formed; all of the order
#   of 1e-6 relative per operation.  Bound: 2e-4 absolute + 2e-4 relative (|logits| ~ 1).
#   bfloat16: both sides round activations to bfloat16 (2^-8 relative) where the engine
#   stores them, but sums run in other orders, so single roundings fall differently, and
#   the tensor-core prompt attention also rounds its probabilities to bfloat16 before the
#   value product.  Such noise scales with the size of the logits, not with the single
#   value, so the bound is stated in units of the largest logit of the tensor:
#   every value within 2^-6 * (max|plain| + |plain|), and the root-mean-square error within
#   2^-8 * max|plain|.  A fault of the cache or the batch (a wrong key, a wrong position, a
#   stale slot) moves logits by tenths of that scale: tests/test_tolerance_teeth.py plants such
#   faults in the plain implementation and checks that this bound refuses each of them.
TOL = {
    "float32": dict(atol=2e-4, rtol=2e-4),
    "bfloat16": dict(scaled=2.0 ** -6, rms=2.0 ** -8),
}


def compare(got, ref, dtype: str, what: str = "") -> None:
    got = torch.as_tensor(np.asarray(got) if not isinstance(got, torch.Tensor) else got).float().cpu()
    ref = torch.as_tensor(ref).float().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    if ref.numel() == 0:
        return
    tol = TOL[dtype]
    err = (got - ref).abs()
    top = ref.abs().max()
    if "scaled" in tol:
        bound = tol["scaled"] * (top + ref.abs())
        rms = err.pow(2).mean().sqrt().item()
        assert rms <= tol["rms"] * top.item(), f"{what}: rms error {rms:.3g} (|plain| max {top.item():.3g})"
    else:
        bound = tol["atol"] + tol["rtol"] * ref.abs()
    if not (err <= bound).all():
        idx = torch.nonzero(err > bound)[0].tolist()
        raise AssertionError(
            f"{what}: {int((err > bound).sum())} of {err.numel()} values differ; first at {idx}: "
            f"got {got[tuple(idx)].item():.6g}, plain {ref[tuple(idx)].item():.6g}; "
            f"max abs err {err.max().item():.3g} (|plain| max {top.item():.3g})")
