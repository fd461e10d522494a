"""Choice of the next token from logits, on the device.

Reference: `sample_greedy` (first largest logit; empty or non-finite logits are an error,
src/engine/sampling.rs:25-49) and `sample_temperature` (softmax(logits / T), a uniform r
in [0, 1), the first id whose running sum exceeds r, else the last id; T must be positive
and finite, :54-79).  The reference takes the caller's generator; here r is one
Philox4x32-10 draw keyed by the seed with counter (request id, step), so a request draws
the same numbers alone and in any batch.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from ..csrc import bindings as B


class SamplingError(ValueError):
    pass


@dataclass(frozen=True)
class SamplingParams:
    """temperature 0 = greedy; > 0 = temperature sampling with `seed`."""
    temperature: float = 0.0
    seed: int = 0

    def __post_init__(self):
        t = self.temperature
        if isinstance(t, bool) or not isinstance(t, (int, float)) or not math.isfinite(t) or t < 0:
            raise SamplingError(f"temperature must be finite and >= 0 (0 = greedy), got {t!r}")
        if isinstance(self.seed, bool) or not isinstance(self.seed, int) or not 0 <= self.seed < 2 ** 64:
            raise SamplingError(f"seed must be an integer in [0, 2^64), got {self.seed!r}")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0


class Sampler:
    """Samples one token per row of a float32 [rows, vocab] logits tensor on the device."""

    def __init__(self, params: SamplingParams, err: torch.Tensor):
        self.params = params
        self.err = err

    def sample_device(self, logits: torch.Tensor, request_ids: Sequence[int],
                      steps: Sequence[int]) -> torch.Tensor:
        """int32 [rows] on the device.  `request_ids[i]`, `steps[i]`: the Philox counter of row i."""
        rows = logits.shape[0]
        if logits.dim() != 2 or rows == 0 or logits.shape[1] == 0:
            raise SamplingError("logits are empty")          # src/engine/sampling.rs:58-60
        if logits.dtype != torch.float32:
            raise SamplingError(f"logits must be float32, got {logits.dtype}")
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
        stream = B.stream_ptr()
        if self.params.greedy:
            B.sample_greedy(logits, out, self.err, stream)
        else:
            if len(request_ids) != rows or len(steps) != rows:
                raise SamplingError("one request id and one step per row are needed")
            ctr = torch.tensor([list(request_ids), list(steps)], dtype=torch.int32).to(logits.device)
            B.sample_temperature(logits, float(self.params.temperature), self.params.seed,
                                 ctr[0], ctr[1], out, self.err, stream)
        return out

    def __call__(self, logits: torch.Tensor, request_ids: Sequence[int], steps: Sequence[int]) -> List[int]:
        """Host token ids (synchronises), after checking the device error word."""
        out = self.sample_device(logits, request_ids, steps)
        tokens = out.tolist()
        bits = int(self.err.item())
        if bits:
            self.err.zero_()
            raise SamplingError(B.describe_error_bits(bits))
        return tokens
