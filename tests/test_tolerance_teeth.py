"""Do the logit tolerances reject real faults?  The plain implementation is run with a fault
planted in it (the kind a cache, a batch or a kernel index would make) and with the rounding
of a bfloat16 engine, and `compare` must refuse the result at the bfloat16 tolerance (and so
at the tighter float32 one), on the tiny configurations and lengths that the GPU tests use,
over all rows of a request at once, as those tests compare them (a fault in one token's row is
not hidden by the rows that are right).

Faults: the window one key wider or narrower; query heads mapped to kv heads by `h % kv_heads`
instead of `h // group`; the last token rotated for the position after its own; for the
configuration without a window, a window where there is none.
"""
import pytest
import torch

from helpers import TINY, WEIGHT_STD, compare, prompts_for
from plain import mistral_plain as P
from inference_engine_rust_b200 import Model, config_from_dict, spec_of
from inference_engine_rust_b200.parts.base import Runtime
from inference_engine_rust_b200.weights import RandomSource


def weights_of(cfg, seed=11):
    model = Model(spec_of(config_from_dict(cfg)), Runtime(dtype=torch.float32, device="cpu"))
    exp = model.expected_tensors()
    src = RandomSource(exp, seed, WEIGHT_STD, dtype=torch.bfloat16)
    return {n: src.get(n).float() for n in exp}


def faults(cfg, T):
    out = {}
    w = cfg.get("sliding_window")
    if w is not None and T > w:
        out["window one wider"] = (dict(cfg, sliding_window=w + 1), {})
        out["window one narrower"] = (dict(cfg, sliding_window=w - 1), {})
    elif w is None and T > 16:
        out["a window of 16 where there is none"] = (dict(cfg, sliding_window=16), {})
    kvh = cfg["num_key_value_heads"]
    group = cfg["num_attention_heads"] // kvh
    if kvh > 1 and group > 1:
        out["kv head of a query head taken modulo"] = (cfg, {"kv_head_of": lambda h: h % kvh})
    out["last token one position late"] = (cfg, {"positions": list(range(T - 1)) + [T]})
    return out


@pytest.mark.parametrize("name,T", [("A", 23), ("A", 70), ("A", 150), ("B", 19), ("B", 40), ("B", 130)])
def test_planted_faults_are_rejected(name, T):
    cfg = TINY[name]
    w = weights_of(cfg)
    ids = prompts_for(cfg, [T], seed=5)[0]
    good = P.forward(cfg, w, ids, P.bf16_rounding)
    # the comparison itself passes for what differs by rounding only
    compare(P.forward(cfg, w, ids, P.no_rounding), good, "bfloat16", "rounding alone")
    planted = faults(cfg, T)
    assert len(planted) >= 2
    for what, (bad_cfg, options) in planted.items():
        bad = P.forward(bad_cfg, w, ids, P.bf16_rounding, **options)
        with pytest.raises(AssertionError):
            compare(bad, good, "bfloat16", what)
        with pytest.raises(AssertionError):
            compare(bad, good, "float32", what)
