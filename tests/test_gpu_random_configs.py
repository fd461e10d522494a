"""Configurations drawn at random (a fixed seed) over every size and option the architecture's
configuration allows: head sizes in steps of 16, any number of heads and groups, widths, feed-forward
sizes and vocabularies that are no power of two, windows that cut pages and tiles at odd places, one
to three layers, tied and untied heads.  Each model is run in 32-bit and in bfloat16 on a batch of
unequal prompts whose last tokens come one by one, and compared with the plain implementation: a
kernel either takes a size or refuses it (and its plain sibling runs), never a wrong result.

A longer hunt (IERT_TEST_RANDOM_CONFIGS=160, 320 cases) passes every 32-bit case; of the bfloat16 cases about
one in thirty has a handful of logits (1 to 18 of tens of thousands) outside the per-value bound, all at wide
models with several layers, where the plain bfloat16 statement itself is 4 to 12 % of the largest logit away
from the 32-bit result: there the engine's error against the 32-bit result equals the plain statement's
(both measured), and the two differ from each other by a quarter of it.  The twelve cases kept here are
within the bound."""
import os

import numpy as np
import pytest
import torch

from helpers import WEIGHT_STD, compare
from plain import mistral_plain as P

pytestmark = pytest.mark.gpu


def draw_config(rng):
    head_dim = int(rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 160, 256]))
    kv = int(rng.choice([1, 2, 3, 4]))
    heads = kv * int(rng.choice([1, 2, 3, 5]))
    hidden = int(rng.choice([40, 72, 104, 136, 200, 264, 328]))
    window = rng.choice([None, 5, 16, 33, 70, 129])
    return {
        "architectures": ["MistralForCausalLM"],
        "num_hidden_layers": int(rng.integers(1, 4)),
        "hidden_size": hidden,
        "num_attention_heads": heads,
        "num_key_value_heads": kv,
        "head_dim": head_dim,
        "intermediate_size": int(rng.choice([40, 88, 136, 200, 296])),
        "vocab_size": int(rng.choice([61, 127, 300, 515, 1001])),
        "rope_theta": float(rng.choice([1e4, 5e5, 1e6])),
        "rms_norm_eps": float(rng.choice([1e-5, 1e-6, 3e-4])),
        "sliding_window": None if window is None else int(window),
        "max_position_embeddings": 512,
        "tie_word_embeddings": bool(rng.integers(0, 2)),
    }


# (more of them for a longer hunt: IERT_TEST_RANDOM_CONFIGS=200)
CONFIGS = [draw_config(np.random.default_rng(1000 + i)) for i in range(int(os.environ.get("IERT_TEST_RANDOM_CONFIGS", "12")))]


def _id(cfg):
    return (f"L{cfg['num_hidden_layers']}-H{cfg['hidden_size']}-h{cfg['num_attention_heads']}x{cfg['num_key_value_heads']}"
            f"-d{cfg['head_dim']}-I{cfg['intermediate_size']}-V{cfg['vocab_size']}-W{cfg['sliding_window']}"
            f"{'-tied' if cfg['tie_word_embeddings'] else ''}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cfg", CONFIGS, ids=_id)
def test_a_random_configuration_against_the_plain_implementation(cfg, dtype):
    from inference_engine_rust_b200 import LoadedModel
    from inference_engine_rust_b200.weights import RandomSource
    seed = 7 + cfg["hidden_size"] + cfg["head_dim"]
    model = LoadedModel.random(cfg, seed=seed, dtype=dtype, std=WEIGHT_STD)
    src = RandomSource(model.model.expected_tensors(), seed, WEIGHT_STD, dtype=torch.float32)
    w = {n: src.get(n) for n in src.names()}
    if dtype == "bfloat16":
        w = {n: t.to(torch.bfloat16).float() for n, t in w.items()}
    if cfg["tie_word_embeddings"]:
        assert "lm_head.weight" not in w
        w["lm_head.weight"] = w["model.embed_tokens.weight"]
    rnd = P.bf16_rounding if dtype == "bfloat16" else P.no_rounding
    rng = np.random.default_rng(seed)
    lengths = [int(rng.integers(1, 8)), int(rng.integers(60, 70)), int(rng.integers(100, 180))]
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in lengths]
    want = [P.forward(cfg, w, p, rnd) for p in prompts]
    eng = model.session(max_tokens=64 * 6, poison_cache=True).engine
    tails = [min(4, n - 1) for n in lengths]
    slots = [eng.open_sequence() for _ in prompts]
    got = [[] for _ in prompts]
    out = eng.step([(s, p[:len(p) - t]) for s, p, t in zip(slots, prompts, tails)], want="all")
    at = 0
    for i, (p, t) in enumerate(zip(prompts, tails)):
        got[i].append(out[at:at + len(p) - t].clone())
        at += len(p) - t
    for k in range(max(tails)):
        live = [i for i in range(len(prompts)) if tails[i] > k]
        out = eng.step([(slots[i], [prompts[i][len(prompts[i]) - tails[i] + k]]) for i in live], want="last")
        for r, i in enumerate(live):
            got[i].append(out[r:r + 1].clone())
    eng.check_device()
    for i in range(len(prompts)):
        try:
            compare(torch.cat(got[i]), want[i], dtype, f"request {i} ({lengths[i]} tokens)")
        except AssertionError as e:
            if dtype != "bfloat16":
                raise
            # for the reader of a failure: how far the engine and the plain bfloat16 statement each are from
            # the 32-bit result (about equal: rounding noise of this configuration; engine far worse: a fault)
            w32 = {n: src.get(n) for n in src.names()}
            if cfg["tie_word_embeddings"]:
                w32["lm_head.weight"] = w32["model.embed_tokens.weight"]
            truth = P.forward(cfg, w32, prompts[i], P.no_rounding)
            def rms(a, b):
                return float((a.float().cpu() - b).pow(2).mean().sqrt())
            raise AssertionError(f"{e}\n(rms distance to the 32-bit result: engine {rms(torch.cat(got[i]), truth):.4g}, "
                                 f"plain bfloat16 statement {rms(want[i], truth):.4g})") from None
