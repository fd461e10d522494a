"""The generation loop above the step function: batches of unequal prompts, stop tokens,
sequences that end earlier than others, and as many batches one after another as there
are requests.

Reference loop (src/main.rs:97-116): prefill the prompt; then up to `new_tokens` times:
choose the next token from the last logits; if it is the stop token, end WITHOUT keeping
it; keep it; run it through the model.  The reference also runs the model on the last kept
token although nothing reads the result; this loop does not.  Policy and loop stay apart
as in src/engine/generation.rs:5-9: `sampler` chooses, this file decides who goes on.

The loop only needs an object with open_sequence(), close_sequence(slot) and
step(entries, want="last") and a callable sampler(logits, request_ids, steps) -> token ids,
so its decisions can be tested without a device.

Where the engine can take a step's tokens from device memory (`step_tokens_on_device`) and the
sampler can hand them back without waiting (`sample_device`, `read_async`), the loop runs one
step ahead of the host: the ids chosen from step k's logits stay on the device and feed step
k + 1 at once, and the host reads them, decides who has ended and calls `on_token` while step
k + 1 runs.  Who goes on by count alone (new-token limit, context) is known beforehand; only a
stop token is not, so a sequence that ends on one has run one step in vain, whose result nobody
reads and whose slot is given back like any other.  Tokens, reasons and the order of `on_token`
calls are those of the plain loop.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, Iterable, List, Optional, Sequence, Set


@dataclass
class GenerationResult:
    request: int                    # index of the request among the prompts given
    prompt_len: int
    tokens: List[int] = field(default_factory=list)   # generated ids, the stop token not among them
    finish_reason: str = ""         # "stop" | "length" | "context"


def plan_batches(prompt_lens: Sequence[int], max_new_tokens: int, *, max_tokens: int,
                 max_sequences: int, max_seq_len: int, page_tokens: int,
                 max_batch: Optional[int] = None) -> List[List[int]]:
    """Split requests, in order, into batches that fit the cache: a request may come to hold
    min(prompt + max_new_tokens, max_seq_len) positions, rounded up to a page."""
    if max_batch is not None and max_batch <= 0:
        raise ValueError("max_batch must be positive")
    limit = min(max_sequences, max_batch) if max_batch else max_sequences
    batches: List[List[int]] = []
    cur: List[int] = []
    cur_tokens = 0
    for i, n in enumerate(prompt_lens):
        if n <= 0:
            raise ValueError(f"request {i}: the prompt is empty")
        if n > max_seq_len:
            raise ValueError(f"request {i}: a prompt of {n} tokens exceeds the longest sequence "
                             f"the cache holds ({max_seq_len})")
        need = min(n + max_new_tokens, max_seq_len)
        need = math.ceil(need / page_tokens) * page_tokens
        if need > max_tokens:
            raise ValueError(f"request {i}: needs room for {need} tokens, the cache holds {max_tokens}")
        if cur and (len(cur) >= limit or cur_tokens + need > max_tokens):
            batches.append(cur)
            cur, cur_tokens = [], 0
        cur.append(i)
        cur_tokens += need
    if cur:
        batches.append(cur)
    return batches


def can_run_ahead(engine, sampler) -> bool:
    return (hasattr(engine, "step_tokens_on_device") and hasattr(sampler, "sample_device")
            and hasattr(sampler, "read_async"))


def _keep(res: GenerationResult, tok: int, max_new_tokens: int, stop_ids: Set[int], max_seq_len: int,
          on_token) -> None:
    """What the loop does with a chosen token (src/main.rs:100-108), and why a sequence ends."""
    if tok in stop_ids:                                 # not kept: src/main.rs:104-106
        res.finish_reason = "stop"
        return
    res.tokens.append(tok)
    if on_token is not None:
        on_token(res.request, tok)
    if len(res.tokens) >= max_new_tokens:
        res.finish_reason = "length"
    elif res.prompt_len + len(res.tokens) > max_seq_len:
        res.finish_reason = "context"                   # no room to run this token


def run_batch_ahead(engine, sampler, prompts: Sequence[Sequence[int]], request_ids: Sequence[int],
                    max_new_tokens: int, stop_ids: Set[int], max_seq_len: int,
                    on_token: Optional[Callable[[int, int], None]] = None) -> List[GenerationResult]:
    """`run_batch` with the device one step ahead of the host (see the head of this file)."""
    results = [GenerationResult(request=r, prompt_len=len(p)) for r, p in zip(request_ids, prompts)]
    if max_new_tokens <= 0:
        for res in results:
            res.finish_reason = "length"
        return results
    slots: List[Optional[int]] = []          # opened one by one inside the try: whatever was opened is given back

    def goes_on_if_kept(res: GenerationResult) -> bool:
        """Will the sequence run its next token, if that token is no stop token?"""
        n = len(res.tokens) + 1
        return n < max_new_tokens and res.prompt_len + n <= max_seq_len

    try:
        for _ in prompts:
            slots.append(engine.open_sequence())
        layout = list(range(len(prompts)))         # batch indices in the row order of `chosen_dev`
        logits = engine.step([(slots[i], list(prompts[i])) for i in layout], want="last")
        step_no = 0
        chosen_dev = sampler.sample_device(logits, [request_ids[i] for i in layout], [step_no] * len(layout))
        pending = sampler.read_async(chosen_dev)
        while True:
            rows = [r for r, i in enumerate(layout) if not results[i].finish_reason and goes_on_if_kept(results[i])]
            ahead = None
            if rows:
                nxt = [layout[r] for r in rows]
                logits = engine.step_tokens_on_device([slots[i] for i in nxt], chosen_dev, rows)
                nxt_dev = sampler.sample_device(logits, [request_ids[i] for i in nxt], [step_no + 1] * len(nxt))
                ahead = (nxt, nxt_dev, sampler.read_async(nxt_dev))
            chosen = pending.wait()
            for i, tok in zip(layout, chosen):
                res = results[i]
                if res.finish_reason:                   # ended on a stop token one step ago: its row ran in vain
                    continue
                _keep(res, int(tok), max_new_tokens, stop_ids, max_seq_len, on_token)
                if res.finish_reason:
                    engine.close_sequence(slots[i])
                    slots[i] = None
            if ahead is None:
                break
            layout, chosen_dev, pending = ahead
            step_no += 1
    finally:
        for s in slots:
            if s is not None:
                engine.close_sequence(s)
    return results


def run_batch(engine, sampler: Callable, prompts: Sequence[Sequence[int]], request_ids: Sequence[int],
              max_new_tokens: int, stop_ids: Set[int], max_seq_len: int,
              on_token: Optional[Callable[[int, int], None]] = None) -> List[GenerationResult]:
    """One batch from its prompts to the end of its last sequence."""
    results = [GenerationResult(request=r, prompt_len=len(p)) for r, p in zip(request_ids, prompts)]
    if max_new_tokens <= 0:
        for res in results:
            res.finish_reason = "length"
        return results
    slots: List[Optional[int]] = []          # opened one by one inside the try: whatever was opened is given back
    live = list(range(len(prompts)))           # indices into this batch, in batch order
    try:
        for _ in prompts:
            slots.append(engine.open_sequence())
        logits = engine.step([(slots[i], list(prompts[i])) for i in live], want="last")
        step_no = 0
        while live:
            chosen = sampler(logits, [request_ids[i] for i in live], [step_no] * len(live))
            going_on, feed = [], []
            for i, tok in zip(live, chosen):
                res = results[i]
                _keep(res, int(tok), max_new_tokens, stop_ids, max_seq_len, on_token)
                if res.finish_reason:
                    engine.close_sequence(slots[i])
                    slots[i] = None
                else:
                    going_on.append(i)
                    feed.append(int(tok))
            live = going_on
            if not live:
                break
            logits = engine.step([(slots[i], [t]) for i, t in zip(live, feed)], want="last")
            step_no += 1
    finally:
        for s in slots:
            if s is not None:
                engine.close_sequence(s)
    return results


def generate(engine, sampler: Callable, prompts: Sequence[Sequence[int]], max_new_tokens: int, *,
             stop_ids: Iterable[int] = (), max_tokens: int, max_sequences: int, max_seq_len: int,
             page_tokens: int, max_batch: Optional[int] = None,
             request_ids: Optional[Sequence[int]] = None,
             on_token: Optional[Callable[[int, int], None]] = None,
             run_ahead: bool = True) -> List[GenerationResult]:
    """All requests, batch after batch, results in the order of `prompts`.  `run_ahead`: keep the
    device one step ahead of the host where engine and sampler allow it."""
    if request_ids is None:
        request_ids = list(range(len(prompts)))
    if len(request_ids) != len(prompts):
        raise ValueError("one request id per prompt is needed")
    stop = set(int(s) for s in stop_ids)
    batches = plan_batches([len(p) for p in prompts], max_new_tokens, max_tokens=max_tokens,
                           max_sequences=max_sequences, max_seq_len=max_seq_len,
                           page_tokens=page_tokens, max_batch=max_batch)
    out: List[Optional[GenerationResult]] = [None] * len(prompts)
    for batch in batches:
        run = run_batch_ahead if run_ahead and can_run_ahead(engine, sampler) else run_batch
        res = run(engine, sampler, [prompts[i] for i in batch], [request_ids[i] for i in batch],
                  max_new_tokens, stop, max_seq_len, on_token)
        for i, r in zip(batch, res):
            r.request = i
            out[i] = r
    return out  # type: ignore[return-value]
