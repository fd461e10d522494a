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
        # page-locked host buffers for the ids on their way back, used in rotation (the generation
        # loop has at most two reads in flight)
        self._host: List[Optional[torch.Tensor]] = [None] * 4
        self._events: list = [None] * 4
        self._turn = 0
        self._ctr_host: List[Optional[torch.Tensor]] = [None] * 4
        self._ctr_events: list = [None] * 4
        self._ctr_turn = 0

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
            ctr = self._counters_to_device(request_ids, steps, logits.device)
            B.sample_temperature(logits, float(self.params.temperature), self.params.seed,
                                 ctr[0], ctr[1], out, self.err, stream)
        return out

    def _counters_to_device(self, request_ids: Sequence[int], steps: Sequence[int], device) -> torch.Tensor:
        """int32 [2, rows] on the device, sent from a page-locked buffer without waiting for the
        device (a copy out of ordinary memory would hold the host until the stream has drained)."""
        rows = len(request_ids)
        i = self._ctr_turn
        self._ctr_turn = (i + 1) % len(self._ctr_host)
        if self._ctr_events[i] is not None:
            self._ctr_events[i].synchronize()          # the copy that last used this buffer is over
        buf = self._ctr_host[i]
        if buf is None or buf.shape[1] < rows:
            buf = self._ctr_host[i] = torch.empty((2, max(rows, 64)), dtype=torch.int32, pin_memory=True)
        view = buf[:, :rows]
        view[0] = torch.tensor(list(request_ids), dtype=torch.int32)
        view[1] = torch.tensor(list(steps), dtype=torch.int32)
        dev = torch.empty((2, rows), dtype=torch.int32, device=device)
        dev.copy_(view, non_blocking=True)
        ev = self._ctr_events[i]
        if ev is None:
            ev = self._ctr_events[i] = torch.cuda.Event()
        ev.record()
        return dev

    def read_async(self, tokens: torch.Tensor) -> "PendingTokens":
        """Start the copy of device token ids (int32 [rows], as `sample_device` returns them) and
        of the device error word to the host, and return at once; `wait()` on the result gives
        the ids.  The caller may launch more work in between: the generation loop starts the
        next step from the ids on the device and reads them on the host one step behind."""
        rows = tokens.shape[0]
        i = self._turn
        self._turn = (i + 1) % len(self._host)
        buf = self._host[i]
        if buf is None or buf.numel() < rows + 1:
            buf = self._host[i] = torch.empty(max(rows + 1, 65), dtype=torch.int32, pin_memory=True)
        buf[:rows].copy_(tokens, non_blocking=True)
        buf[rows:rows + 1].copy_(self.err, non_blocking=True)
        ev = self._events[i]
        if ev is None:
            ev = self._events[i] = torch.cuda.Event()
        ev.record()
        return PendingTokens(self, buf, rows, ev)

    def __call__(self, logits: torch.Tensor, request_ids: Sequence[int], steps: Sequence[int]) -> List[int]:
        """Host token ids (synchronises), after checking the device error word."""
        return self.read_async(self.sample_device(logits, request_ids, steps)).wait()


class PendingTokens:
    """Token ids on their way to the host (one copy for the ids and the error word, one wait)."""

    def __init__(self, sampler: Sampler, buf: torch.Tensor, rows: int, event):
        self._sampler, self._buf, self._rows, self._event = sampler, buf, rows, event

    def wait(self) -> List[int]:
        """The ids, after checking the device error word as it stood when they were chosen."""
        self._event.synchronize()
        values = self._buf[:self._rows + 1].tolist()
        bits = values.pop()
        if bits:
            self._sampler.err.zero_()
            raise SamplingError(B.describe_error_bits(bits))
        return values
