"""Latency and throughput of one model folder, in the reference's terms
(src/bench_metrics.rs, src/bin/bench_compare.rs): cold start through the first token, time to
the first token with warm weights and a fresh cache, and greedy decode throughput after a warm
prefill.  Every figure is wall-clock time on the host around calls of the public entry point
(`LoadedModel`, `InferenceSession`), with the device drained at each boundary, so it includes
what a user of the library pays.

What has no counterpart here is left out rather than reported as zero: the tokenizer timings
(token ids come in), `gguf_metadata_ms` / `weights_build_ms` (a folder is read in one pass:
`config_ms` and `tensor_load_ms`), and the llama.cpp comparison.
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional, Sequence

DEFAULT_BENCH_PROMPT = [1, 415, 7, 88, 9, 13]       # six ids, as long as the reference's default prompt


def _now() -> float:
    return time.perf_counter()


def _sync() -> None:
    import torch
    if torch.cuda.is_available():
        torch.cuda.synchronize()


def _ms(t0: float) -> float:
    return (time.perf_counter() - t0) * 1e3


def _first_token(session, logits) -> List[int]:
    """Greedy choice for every sequence of the batch, read back to the host."""
    from .sampling import Sampler, SamplingParams
    n = logits.shape[0]
    sampler = Sampler(SamplingParams(temperature=0.0), session.engine.rt.err)
    return sampler(logits, list(range(n)), [0] * n)


def run_cold_start(model_dir: str, prompt: Sequence[int], dtype: str = "bfloat16", batch: int = 1,
                   max_tokens: Optional[int] = None):
    """From the folder on disk to the first greedy token id (src/bench_metrics.rs:199-296).
    Returns the metrics and the loaded model, warm, for the runs that follow."""
    from .api import LoadedModel
    from .config import load_config
    wall0 = _now()
    t0 = _now()
    load_config(model_dir)
    config_ms = _ms(t0)
    t0 = _now()
    loaded = LoadedModel.load(model_dir, dtype=dtype)
    _sync()
    tensor_load_ms = _ms(t0)
    t0 = _now()
    session = loaded.session(max_tokens=max_tokens or _cache_tokens(len(prompt), 1, batch), max_sequences=batch)
    _sync()
    kv_alloc_ms = _ms(t0)
    t0 = _now()
    logits = session.prefill([list(prompt)] * batch)
    _sync()
    prompt_eval_ms = _ms(t0)
    t0 = _now()
    _first_token(session, logits)
    lm_head_sample_ms = _ms(t0)
    cold_ttft_ms = _ms(wall0)
    session.reset()
    return {
        "prompt_token_count": len(prompt), "batch": batch, "config_ms": config_ms, "tensor_load_ms": tensor_load_ms,
        "kv_alloc_ms": kv_alloc_ms, "prompt_eval_ms": prompt_eval_ms, "lm_head_sample_ms": lm_head_sample_ms,
        "cold_ttft_ms": cold_ttft_ms,
    }, loaded


def _cache_tokens(prompt_len: int, new_tokens: int, batch: int) -> int:
    return batch * (-(-(prompt_len + new_tokens + 1) // 64) * 64)


class EngineBench:
    """A loaded model and the two warm measurements (src/bench_metrics.rs:87-196)."""

    def __init__(self, loaded, batch: int = 1):
        self.loaded = loaded
        self.batch = batch
        self._sess = None

    @classmethod
    def load(cls, model_dir: str, dtype: str = "bfloat16", batch: int = 1) -> "EngineBench":
        from .api import LoadedModel
        return cls(LoadedModel.load(model_dir, dtype=dtype), batch)

    def _session(self, prompt_len: int, new_tokens: int):
        """One session for all runs of this bench (its cache is given back between runs), so that
        what the engine sets up once per shape (captured graphs) is set up once, as in a server
        that answers request after request."""
        need = _cache_tokens(prompt_len, new_tokens, self.batch)
        if self._sess is None or self._sess.max_tokens < need:
            self._sess = self.loaded.session(max_tokens=need, max_sequences=self.batch)
        self._sess.reset()
        return self._sess

    def run_interactive_ttft(self, prompt: Sequence[int]) -> Dict[str, float]:
        """Warm weights, fresh cache slots: prompt evaluation, then the choice of the first token.
        The final norm and the output projection of the prompt's last token run inside the
        prefill step here, so `lm_head_sample_ms` is the sampling kernel and the read-back alone."""
        session = self._session(len(prompt), 1)
        _sync()
        t0 = _now()
        logits = session.prefill([list(prompt)] * self.batch)
        _sync()
        prompt_eval_ms = _ms(t0)
        t0 = _now()
        _first_token(session, logits)
        lm_head_sample_ms = _ms(t0)
        session.reset()
        return {"prompt_token_count": len(prompt), "batch": self.batch, "prompt_eval_ms": prompt_eval_ms,
                "lm_head_sample_ms": lm_head_sample_ms, "ttft_infer_ms": prompt_eval_ms + lm_head_sample_ms}

    def run_decode_throughput(self, prompt: Sequence[int], decode_tokens: int) -> Dict[str, float]:
        """`decode_tokens` full greedy steps after a warm prefill: choose the next token from the
        last logits, read it back, feed it (src/bench_metrics.rs:158-195, the loop of
        src/main.rs).  With a batch, every sequence decodes and tokens/s counts them all."""
        if decode_tokens <= 0:
            raise ValueError("decode_throughput: decode_tokens must be > 0")
        from .sampling import Sampler, SamplingParams
        n = self.batch
        session = self._session(len(prompt), decode_tokens)
        sampler = Sampler(SamplingParams(temperature=0.0), session.engine.rt.err)
        _sync()
        t0 = _now()
        logits = session.prefill([list(prompt)] * n)
        _sync()
        warm_prefill_ms = _ms(t0)
        reqs = list(range(n))
        t0 = _now()
        # as the generation loop runs it: the chosen ids feed the next step from device memory and
        # are read on the host, every step, while that step runs
        chosen = sampler.sample_device(logits, reqs, [0] * n)
        pending = sampler.read_async(chosen)
        for i in range(decode_tokens):
            logits = session.decode_tokens_on_device(chosen)
            pending.wait()
            if i + 1 < decode_tokens:
                chosen = sampler.sample_device(logits, reqs, [i + 1] * n)
                pending = sampler.read_async(chosen)
        _sync()
        decode_elapsed_ms = _ms(t0)
        session.engine.check_device()
        session.reset()
        return {"prompt_token_count": len(prompt), "batch": n, "decode_tokens": decode_tokens,
                "warm_prefill_ms": warm_prefill_ms, "decode_elapsed_ms": decode_elapsed_ms,
                "decode_tokens_per_sec": n * decode_tokens / max(decode_elapsed_ms / 1e3, 1e-12)}


def run_all(model_dir: str, prompt: Sequence[int], decode_tokens: int, dtype: str = "bfloat16", batch: int = 1):
    """Cold start, then interactive TTFT and decode throughput on the now warm model, in one
    process (src/bench_metrics.rs:298-318)."""
    cold, loaded = run_cold_start(model_dir, prompt, dtype=dtype, batch=batch)
    bench = EngineBench(loaded, batch)
    return {"cold": cold, "interactive": bench.run_interactive_ttft(prompt),
            "decode": bench.run_decode_throughput(prompt, decode_tokens)}


# ---- summaries over runs (src/bin/bench_compare.rs:234-300) ---------------------------------

def median(values: Sequence[float]) -> float:
    v = sorted(values)
    if not v:
        return 0.0
    mid = len(v) // 2
    return v[mid] if len(v) % 2 else (v[mid - 1] + v[mid]) / 2.0


def percentile(values: Sequence[float], p: float) -> float:
    """The value at rank round((n - 1) * p) of the sorted values."""
    v = sorted(values)
    if not v:
        return 0.0
    return v[int((len(v) - 1) * p + 0.5)]


def _spread(values: Sequence[float], with_p95: bool = False) -> Dict[str, float]:
    out = {"median": median(values)}
    if with_p95:
        out["p95"] = percentile(values, 0.95)
    out["min"] = min(values)
    out["max"] = max(values)
    return out


def summarize_interactive(runs: Sequence[Dict[str, float]]) -> Dict[str, object]:
    if not runs:
        raise ValueError("interactive runs are empty")
    return {"runs": len(runs), "ttft_infer_ms": _spread([r["ttft_infer_ms"] for r in runs]),
            "prompt_eval_ms": _spread([r["prompt_eval_ms"] for r in runs])}


def summarize_decode(runs: Sequence[Dict[str, float]]) -> Dict[str, object]:
    if not runs:
        raise ValueError("decode runs are empty")
    return {"runs": len(runs),
            "decode_tokens_per_sec": _spread([r["decode_tokens_per_sec"] for r in runs], with_p95=True),
            "decode_elapsed_ms": _spread([r["decode_elapsed_ms"] for r in runs])}


def check_decode(m: Dict[str, float], min_tps: Optional[float]) -> None:
    """The reference's acceptance of a decode run (src/bin/bench_compare.rs:123-143)."""
    import math
    if not math.isfinite(m["decode_tokens_per_sec"]) or not math.isfinite(m["decode_elapsed_ms"]):
        raise RuntimeError("decode.decode_tokens_per_sec is not finite")
    if m["decode_tokens"] == 0:
        raise RuntimeError("decode.decode_tokens is zero")
    if min_tps is not None and m["decode_tokens_per_sec"] < min_tps:
        raise RuntimeError(f"decode.decode_tokens_per_sec {m['decode_tokens_per_sec']:.3f} < --min-decode-tps {min_tps:.3f}")
