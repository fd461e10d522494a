"""Writes `plain_tiny_logits.npz`: logits of the plain implementation (tests/plain) for the tiny
configurations A and B with seeded random weights and seeded token ids.

These are NOT outputs of the reference: the reference is a Rust crate that cannot be built or run
here, so the plain implementation rests on its formulas (each function cites the lines) and on the
numeric vectors of the reference's unit tests (tests/test_plain.py).  The file pins the plain
implementation against accidental change: tests/test_plain.py recomputes and compares.

    python tests/golden/make_golden.py        # from the repository root
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))


def compute():
    import torch
    from helpers import TINY, prompts_for
    from plain import mistral_plain as P
    from inference_engine_rust_b200.engine.model import Model            # only for the tensor names and shapes
    from inference_engine_rust_b200.config import config_from_dict, spec_of
    from inference_engine_rust_b200.weights import RandomSource
    from inference_engine_rust_b200.parts.base import Runtime
    out = {}
    for name, lengths in (("A", [23]), ("B", [19])):
        cfg = TINY[name]
        model = Model(spec_of(config_from_dict(dict(cfg))), Runtime(dtype=torch.float32, device="cpu"))
        src = RandomSource(model.expected_tensors(), 7, 0.1, dtype=torch.float32)
        w = {n: src.get(n).float() for n in src.names()}
        ids = prompts_for(cfg, lengths, seed=3)[0]
        out[f"{name}_ids"] = np.asarray(ids, dtype=np.int32)
        out[f"{name}_logits"] = P.forward(cfg, w, ids).numpy().astype(np.float32)
    return out


if __name__ == "__main__":
    data = compute()
    path = os.path.join(HERE, "plain_tiny_logits.npz")
    np.savez_compressed(path, **data)
    print(path, {k: v.shape for k, v in data.items()}, os.path.getsize(path), "bytes")
