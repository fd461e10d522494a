"""The step function: one batch of sequences, either all at their first token (prompts of
unequal lengths, packed back to back) or all bringing one more token, run through the
model against the cache.  It runs exactly the tokens it is given and returns the logits at
the wanted places.

Reference: `InferenceSession::prefill` / `decode_token` / `logits_last_token`
(src/engine/session.rs:44-74) for one sequence; the host-side checks are the reference's
error classes (empty prompt and too-long prompt src/engine/embed.rs:109-118, token out of
vocabulary src/layers/embeddings.rs:119-126, cache full src/layers/attention.rs:55-59),
raised here before anything is launched.
"""
from __future__ import annotations

import contextlib
import gc
from typing import List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from ..cache import PAGE_TOKENS, Cache, CacheError, CacheFull
from ..csrc import bindings as B
from ..parts.base import HostCopyUnavailable, StepContext
from .model import Model


class StepError(ValueError):
    """A step that cannot run as asked (checked on the host; nothing was launched)."""


class DeviceFault(RuntimeError):
    """A kernel reported a problem through the device error word."""


Want = Union[str, Sequence[Sequence[int]], None]


class _Staging:
    """Pinned host buffers for a step's integer metadata, used in rotation so that a buffer
    is rewritten only after its copy to the device has finished."""

    def __init__(self, device, depth: int = 4):
        self.device = device
        self.depth = depth
        self.host: List[Optional[torch.Tensor]] = [None] * depth
        self.events: List[Optional[torch.cuda.Event]] = [None] * depth
        self.turn = 0

    def next(self, n_ints: int) -> Tuple[torch.Tensor, int]:
        i = self.turn
        self.turn = (self.turn + 1) % self.depth
        if self.events[i] is not None:
            self.events[i].synchronize()
        buf = self.host[i]
        if buf is None or buf.numel() < n_ints:
            buf = torch.empty(max(n_ints, 4096), dtype=torch.int32, pin_memory=True)
            self.host[i] = buf
        return buf, i

    def sent(self, i: int) -> None:
        ev = self.events[i] or torch.cuda.Event()
        ev.record()
        self.events[i] = ev


@contextlib.contextmanager
def _no_collection_while_capturing():
    """Python's cyclic garbage collector may run at any allocation.  If it then destroys CUDA objects of an
    engine that is no longer used (its graphs, its page-locked staging buffers) while this thread's stream
    is capturing, the CUDA calls in their destructors fail and the process aborts.  Collect before the
    capture and keep the collector off until it has ended."""
    was_enabled = gc.isenabled()
    gc.collect()
    gc.disable()
    try:
        yield
    finally:
        if was_enabled:
            gc.enable()


class _DecodeGraph:
    """A captured one-token step for `nb` sequences: its own metadata buffer, workspace and
    logits buffer (a graph replays fixed addresses), and the graph."""

    def __init__(self, engine: "Engine", nb: int, unequal: bool = False):
        rt, model = engine.rt, engine.model
        from ..parts.base import Workspace
        _, o_slot, _, o_seq, o_tok, o_rows, total = Engine._layout(nb, nb, nb)
        self.meta = torch.zeros(total, dtype=torch.int32, device=rt.device)
        self.meta[o_slot:o_slot + nb] = -1            # all padding until a step fills it in
        self.meta[o_seq:o_seq + nb] = -1
        self.meta[0:nb + 1] = torch.arange(nb + 1, dtype=torch.int32)
        self.meta[o_rows:o_rows + nb] = torch.arange(nb, dtype=torch.int32)
        self.logits = torch.empty((nb, model.spec.vocab_size), dtype=torch.float32, device=rt.device)
        self.ws = Workspace(rt.device)
        self.graph = torch.cuda.CUDAGraph()
        saved = rt.workspace
        rt.workspace = self.ws
        try:
            def run():
                # the launches are replayed for other sequences: their host lists must not be read
                ctx = engine._context("decode", self.meta, nb, nb, [1] * nb, HostCopyUnavailable("pos0"),
                                      HostCopyUnavailable("slots"))
                ctx.unequal_lengths = unequal
                model.forward(ctx, self.meta[o_tok:o_tok + nb], engine.cache,
                              self.meta[o_rows:o_rows + nb], nb, logits_out=self.logits)
            run()                                      # eager once: lazy set-up happens outside the capture
            torch.cuda.synchronize()
            before = B.launch_count
            with _no_collection_while_capturing(), torch.cuda.graph(self.graph):
                run()
            self.launches = B.launch_count - before    # kernels one replay launches
        finally:
            rt.workspace = saved


class _PromptGraph:
    """A captured prompt step for up to `nb` sequences and `tb` tokens in all (short prompts,
    where launching a few hundred kernels costs the host more than they cost the device).
    Tokens beyond the step's own are padding (sequence -1) and sequences beyond its own have
    slot -1: every kernel skips them, so padding changes no result."""

    def __init__(self, engine: "Engine", nb: int, tb: int):
        rt, model = engine.rt, engine.model
        from ..parts.base import Workspace
        self.nb, self.tb = nb, tb
        _, o_slot, _, o_seq, o_tok, o_rows, total = Engine._layout(nb, tb, nb)
        self.meta = torch.zeros(total, dtype=torch.int32, device=rt.device)
        self.meta[o_slot:o_slot + nb] = -1            # all padding until a step fills it in
        self.meta[o_seq:o_seq + tb] = -1
        self.logits = torch.empty((nb, model.spec.vocab_size), dtype=torch.float32, device=rt.device)
        self.ws = Workspace(rt.device)
        self.graph = torch.cuda.CUDAGraph()
        saved = rt.workspace
        rt.workspace = self.ws
        try:
            def run():
                # launches are sized for the longest prompt the bucket can hold
                # (prompts all start at position 0; which slots they are is not known here)
                ctx = engine._context("prompt", self.meta, nb, tb, [tb] + [0] * (nb - 1), [0] * nb,
                                      HostCopyUnavailable("slots"))
                model.forward(ctx, self.meta[o_tok:o_tok + tb], engine.cache,
                              self.meta[o_rows:o_rows + nb], nb, logits_out=self.logits)
            run()                                      # eager once: lazy set-up happens outside the capture
            torch.cuda.synchronize()
            before = B.launch_count
            with _no_collection_while_capturing(), torch.cuda.graph(self.graph):
                run()
            self.launches = B.launch_count - before
        finally:
            rt.workspace = saved


PROMPT_GRAPH_MAX_TOKENS = 512       # longer prompts keep the device busy enough when launched one by one
PROMPT_GRAPH_MAX_SEQUENCES = 8


class Engine:
    """A model, its cache, and the step function over them."""

    def __init__(self, model: Model, *, max_tokens: int, max_sequences: Optional[int] = None,
                 max_seq_len: Optional[int] = None, poison_cache: bool = False, use_graphs: bool = True,
                 page_tokens: int = PAGE_TOKENS):
        if not model.loaded:
            raise ValueError("the model has no weights yet (load() or load_random() first)")
        B.require_device()
        self.model = model
        self.rt = model.rt
        spec = model.spec
        n_pages = -(-max_tokens // page_tokens)
        if max_sequences is None:
            max_sequences = max(1, min(n_pages, 1024))
        if max_seq_len is None:
            max_seq_len = spec.max_position
        self.cache = Cache(model.cache_requests(), max_tokens=max_tokens,
                           max_seq_len=min(max_seq_len, spec.max_position),
                           max_sequences=max_sequences, dtype=self.rt.dtype, device=self.rt.device,
                           page_tokens=page_tokens, poison=poison_cache)
        self._staging = _Staging(self.rt.device)
        self._meta_dev: Optional[torch.Tensor] = None
        self.steps_run = 0
        self.h2d_bytes_last_step = 0
        self.graph_launches = 0        # kernels launched by graph replays so far
        # one-token steps replay captured graphs when every part of the model says that its
        # forward depends on the step only through device memory
        self.use_graphs = use_graphs and model.graph_safe()
        self._graphs = {}
        self._prompt_uses = {}

    # ---- sequences ------------------------------------------------------------------------
    def open_sequence(self) -> int:
        return self.cache.open_sequence()

    def close_sequence(self, slot: int) -> None:
        self.cache.close_sequence(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    # ---- the step ---------------------------------------------------------------------------
    def plan(self, entries: Sequence[Tuple[int, Sequence[int]]], want: Want):
        """Host-side checks and the packed description of a step.  Launches nothing."""
        spec = self.model.spec
        if not entries:
            raise StepError("a step needs at least one sequence")
        slots = [int(s) for s, _ in entries]
        if len(set(slots)) != len(slots):
            raise StepError("a slot appears twice in one step")
        q_lens, pos0 = [], []
        for slot, toks in entries:
            if len(toks) == 0:
                raise StepError(f"slot {slot}: no tokens (an empty prompt cannot be run)")
            try:
                pos0.append(self.cache.length(slot))
            except CacheError as e:
                raise StepError(str(e)) from None
            q_lens.append(len(toks))
        if all(q == 1 for q in q_lens):
            kind = "decode"
        elif all(p == 0 for p in pos0):
            kind = "prompt"
        else:
            raise StepError("the sequences of a step must all start at their first token or all "
                            "bring exactly one token")
        tokens = np.fromiter((t for _, toks in entries for t in toks), dtype=np.int64,
                             count=sum(q_lens))
        if tokens.size and (tokens.min() < 0 or tokens.max() >= spec.vocab_size):
            bad = int(tokens[(tokens < 0) | (tokens >= spec.vocab_size)][0])
            raise StepError(f"token id {bad} is outside the vocabulary [0, {spec.vocab_size})")
        for slot, p, q in zip(slots, pos0, q_lens):
            if p + q > self.cache.max_seq_len:
                raise CacheFull(f"slot {slot}: {p + q} tokens exceed the longest sequence the cache "
                                f"holds ({self.cache.max_seq_len})")
        cu = np.zeros(len(entries) + 1, dtype=np.int64)
        np.cumsum(q_lens, out=cu[1:])
        rows: List[int] = []
        if want is None or want == "none":
            pass
        elif want == "last":
            rows = [int(c) - 1 for c in cu[1:]]
        elif want == "all":
            rows = list(range(int(cu[-1])))
        else:
            if len(want) != len(entries):
                raise StepError("`want` needs one list of places per sequence")
            for i, places in enumerate(want):
                for p in places:
                    if not 0 <= p < q_lens[i]:
                        raise StepError(f"wanted place {p} is outside sequence {i}'s {q_lens[i]} tokens")
                    rows.append(int(cu[i]) + int(p))
        return kind, slots, q_lens, pos0, tokens, cu, rows

    def step(self, entries: Sequence[Tuple[int, Sequence[int]]], want: Want = "last"
             ) -> Optional[torch.Tensor]:
        """Run one step.  `entries` = [(slot, tokens)]; `want` = "last", "all", "none"/None, or
        for each sequence the places among its tokens whose logits are wanted.  Returns
        float32 [wanted, vocab] on the device, in the order of the entries and of `want`."""
        plan = self._plan_one_token(entries, want)
        return self._run(plan if plan is not None else self.plan(entries, want), None)

    def _plan_one_token(self, entries, want: Want):
        """`plan` for the step that is run thousands of times in a row: every sequence brings one token
        and the logits of all (or none) are wanted.  The same checks, without the general
        bookkeeping; None where the general plan has to decide (or to raise)."""
        if not entries or not (want == "last" or want == "all" or want is None or want == "none"):
            return None
        held, lens, vocab, limit = self.cache.slots._held, self.cache.seq_lens, self.model.spec.vocab_size, self.cache.max_seq_len
        slots, pos0, toks = [], [], []
        for slot, t in entries:
            if len(t) != 1 or slot not in held:
                return None
            tok, p = t[0], int(lens[slot])
            if not 0 <= tok < vocab or p + 1 > limit:
                return None
            slots.append(int(slot)); pos0.append(p); toks.append(tok)
        n = len(slots)
        if len(set(slots)) != n:
            return None
        rows = list(range(n)) if want in ("last", "all") else []
        return "decode", slots, [1] * n, pos0, toks, range(n + 1), rows

    def step_tokens_on_device(self, slots: Sequence[int], tokens: torch.Tensor,
                              rows: Optional[Sequence[int]] = None, want: Want = "last") -> Optional[torch.Tensor]:
        """A one-token step whose token ids are already on the device: sequence j brings
        `tokens[rows[j]]` (`rows` defaults to 0, 1, ...; int32, for instance straight from the
        sampling kernel).  Nothing waits for the ids on the host, so the step can be launched while
        the step before it still runs; the embedding kernel reports an id outside the vocabulary
        through the device error word."""
        n = len(slots)
        rows = list(range(n)) if rows is None else [int(r) for r in rows]
        if (tokens.dim() != 1 or tokens.dtype != torch.int32 or tokens.device.type != self.rt.device.type
                or len(rows) != n or any(not 0 <= r < tokens.shape[0] for r in rows)):
            raise StepError("device tokens must be int32 [rows] on the model's device, one row per sequence")
        entries = [(s, (0,)) for s in slots]
        plan = self._plan_one_token(entries, want) or self.plan(entries, want)
        if plan[0] != "decode":
            raise StepError("tokens on the device can only continue running sequences by one token")
        return self._run(plan, (tokens, rows))

    def _run(self, plan, device_tokens) -> Optional[torch.Tensor]:
        kind, slots, q_lens, pos0, tokens, cu, rows = plan
        n, T, R = len(slots), int(cu[-1]), len(rows)
        for slot, p, q in zip(slots, pos0, q_lens):
            self.cache.reserve(slot, p + q)
        self.cache.upload()
        if kind == "decode" and self.use_graphs and R in (0, n) and rows == list(range(R)):
            logits = self._step_graph(slots, pos0, tokens, R, device_tokens)
        elif (kind == "prompt" and self.use_graphs and T <= PROMPT_GRAPH_MAX_TOKENS and n <= PROMPT_GRAPH_MAX_SEQUENCES
              and R in (0, n) and rows == [int(c) - 1 for c in cu[1:1 + R]] and self._prompt_bucket_is_warm(n, T)):
            logits = self._step_prompt_graph(slots, q_lens, tokens, cu, R)
        else:
            logits = self._step_eager(kind, slots, q_lens, pos0, tokens, cu, rows, device_tokens)
        for slot, q in zip(slots, q_lens):
            self.cache.advance(slot, q)
        self.steps_run += 1
        return logits

    @staticmethod
    def _layout(n: int, T: int, R: int):
        """Offsets of cu_q | slot_ids | pos0 | tok_seq | tokens | logit_rows in the packed
        integer metadata of a step, and its total length."""
        o_cu, o_slot, o_pos = 0, n + 1, 2 * n + 1
        o_seq, o_tok, o_rows = 3 * n + 1, 3 * n + 1 + T, 3 * n + 1 + 2 * T
        return o_cu, o_slot, o_pos, o_seq, o_tok, o_rows, o_rows + max(R, 1)

    def _context(self, kind, meta, n, T, q_lens, pos0, slots) -> StepContext:
        o_cu, o_slot, o_pos, o_seq, o_tok, o_rows, _ = self._layout(n, T, 0)
        base = meta.data_ptr()
        batch = B.BatchView(cu_q=base + 4 * o_cu, slot_ids=base + 4 * o_slot, tok_seq=base + 4 * o_seq,
                            pos0=base + 4 * o_pos, n_seqs=n, n_tokens=T)
        return StepContext(kind=kind, batch=batch, n_tokens=T, n_seqs=n, q_lens=q_lens, pos0=pos0,
                           slots=slots, stream=B.stream_ptr(), rt=self.rt,
                           slot_ids_dev=meta[o_slot:o_slot + n], pos0_dev=meta[o_pos:o_pos + n],
                           cu_q_dev=meta[o_cu:o_cu + n + 1])

    def _unequal(self, pos0) -> bool:
        """Do the mixers want this one-token step cut by the sequences' lengths?  Steps of either
        kind replay a graph of their own."""
        return len(pos0) >= 2 and self.model.cut_by_length(pos0, self.cache)

    @staticmethod
    def _place_device_tokens(dest: torch.Tensor, device_tokens) -> None:
        """dest[j] = tokens[rows[j]] by one device-to-device copy per run of consecutive rows
        (usually one: rows leave the batch only when a sequence ends)."""
        tokens, rows = device_tokens
        j = 0
        while j < len(rows):
            k = j + 1
            while k < len(rows) and rows[k] == rows[k - 1] + 1:
                k += 1
            dest[j:k].copy_(tokens[rows[j]:rows[j] + (k - j)], non_blocking=True)
            j = k

    def _step_eager(self, kind, slots, q_lens, pos0, tokens, cu, rows, device_tokens=None):
        n, T, R = len(slots), int(cu[-1]), len(rows)
        o_cu, o_slot, o_pos, o_seq, o_tok, o_rows, total = self._layout(n, T, R)
        host, turn = self._staging.next(total)
        h = host.numpy()
        h[o_cu:o_cu + n + 1] = cu
        h[o_slot:o_slot + n] = slots
        h[o_pos:o_pos + n] = pos0
        h[o_seq:o_seq + T] = np.repeat(np.arange(n, dtype=np.int32), q_lens)
        h[o_tok:o_tok + T] = tokens
        h[o_rows:o_rows + R] = rows
        if self._meta_dev is None or self._meta_dev.numel() < total:
            self._meta_dev = torch.empty(max(total, 4096), dtype=torch.int32, device=self.rt.device)
        meta = self._meta_dev
        meta[:total].copy_(host[:total], non_blocking=True)
        self._staging.sent(turn)
        if device_tokens is not None:
            self._place_device_tokens(meta[o_tok:o_tok + T], device_tokens)
        self.h2d_bytes_last_step = total * 4
        ctx = self._context(kind, meta, n, T, q_lens, pos0, slots)
        ctx.unequal_lengths = kind == "decode" and self._unequal(pos0)
        return self.model.forward(ctx, meta[o_tok:o_tok + T], self.cache,
                                  meta[o_rows:o_rows + R] if R else None, R)

    # ---- one-token steps as replayed CUDA graphs ---------------------------------------------
    def _step_graph(self, slots, pos0, tokens, R, device_tokens=None):
        """A one-token step through a captured graph.  Batches are padded to the next power of
        two with sequences whose slot is -1: kernels skip them, so padding changes no result.
        The graph writes its logits into a buffer of its own; the caller gets a copy."""
        n = len(slots)
        nb = 1
        while nb < n:
            nb *= 2
        unequal = self._unequal(pos0)
        g = self._graphs.get((nb, unequal))
        if g is None:
            g = self._graphs[(nb, unequal)] = _DecodeGraph(self, nb, unequal)
        o_cu, o_slot, o_pos, o_seq, o_tok, o_rows, total = self._layout(nb, nb, nb)
        host, turn = self._staging.next(total)
        pad = nb - n
        # cu_q | slot_ids | pos0 | tok_seq | tokens | logit_rows, padding sequences with slot and sequence -1
        host.numpy()[:total] = (list(range(nb + 1)) + list(slots) + [-1] * pad + list(pos0) + [0] * pad
                                + list(range(n)) + [-1] * pad + [int(t) for t in tokens] + [0] * pad + list(range(nb)))
        g.meta[:total].copy_(host[:total], non_blocking=True)
        self._staging.sent(turn)
        if device_tokens is not None:
            self._place_device_tokens(g.meta[o_tok:o_tok + n], device_tokens)
        self.h2d_bytes_last_step = total * 4
        g.graph.replay()
        self.graph_launches += g.launches
        return g.logits[:n].clone() if R else None

    @staticmethod
    def _token_bucket(T: int) -> int:
        """Padded token count of a short prompt step: 16, 32, then multiples of 64 (the token tiles
        of the projection kernel)."""
        return 16 if T <= 16 else 32 if T <= 32 else -(-T // 64) * 64

    def _prompt_bucket_is_warm(self, n: int, T: int) -> bool:
        """A bucket of prompt shapes gets its graph when it is used for the second time: a
        session that runs one prompt and is dropped never pays for a capture."""
        nb = 1
        while nb < n:
            nb *= 2
        key = ("prompt", nb, self._token_bucket(T))
        if key in self._graphs:
            return True
        self._prompt_uses[key] = self._prompt_uses.get(key, 0) + 1
        return self._prompt_uses[key] >= 2

    def _step_prompt_graph(self, slots, q_lens, tokens, cu, R):
        """A short prompt step through a captured graph: sequences padded to a power of two, tokens
        to a multiple of 64; logits at each prompt's last token (or none)."""
        n, T = len(slots), int(cu[-1])
        nb = 1
        while nb < n:
            nb *= 2
        tb = self._token_bucket(T)
        g = self._graphs.get(("prompt", nb, tb))
        if g is None:
            g = self._graphs[("prompt", nb, tb)] = _PromptGraph(self, nb, tb)
        o_cu, o_slot, o_pos, o_seq, o_tok, o_rows, total = self._layout(nb, tb, nb)
        host, turn = self._staging.next(total)
        h = host.numpy()
        h[o_cu:o_cu + n + 1] = cu
        h[o_cu + n + 1:o_cu + nb + 1] = T              # padding sequences are empty
        h[o_slot:o_slot + nb] = -1
        h[o_slot:o_slot + n] = slots
        h[o_pos:o_pos + nb] = 0
        h[o_seq:o_seq + tb] = -1
        h[o_seq:o_seq + T] = np.repeat(np.arange(n, dtype=np.int32), q_lens)
        h[o_tok:o_tok + tb] = 0
        h[o_tok:o_tok + T] = tokens
        h[o_rows:o_rows + nb] = 0
        h[o_rows:o_rows + n] = cu[1:] - 1
        g.meta[:total].copy_(host[:total], non_blocking=True)
        self._staging.sent(turn)
        self.h2d_bytes_last_step = total * 4
        g.graph.replay()
        self.graph_launches += g.launches
        return g.logits[:n].clone() if R else None

    def check_device(self) -> None:
        """Read the device error word (synchronises) and raise if a kernel set a bit."""
        bits = int(self.rt.err.item())
        if bits:
            self.rt.err.zero_()
            raise DeviceFault(B.describe_error_bits(bits))
