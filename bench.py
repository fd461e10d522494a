"""Decode and prefill throughput of the library at Mistral-7B-v0.1 layer sizes with random
weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  A "step" is one decode step of the whole batch (default batch 8 at
2,048 tokens of context, cache sized for 4,096): `value` is decoded tokens a second over K
steps timed with CUDA events on the launching stream (each step = metadata copy, the
captured forward graph, the sampling kernel); `e2e` is the same through the Python entry
point with host token ids in and out every step (`run_ahead_value`: with the chosen ids fed from
device memory and read on the host one step behind, as the library's generation loop does).  Also reported: a 2,048-token prefill
with its fraction of the bf16 tensor peak, the decode step's fraction of the HBM roofline
(every weight once plus the live requests' keys and values, over the step time), and decode
at batch 1 and 64.  Peaks come from MEASURED_PEAKS.json when the driver wrote it.

The method follows the reference's own bench (src/bench_metrics.rs:158-195): an untimed warm
prefill, then a timed loop of full decode steps including the choice of the next token.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Layer sizes of Mistral 7B v0.1 (the benchmark configuration; the library itself takes
# every size from config.json).
MISTRAL_7B = {
    "architectures": ["MistralForCausalLM"], "model_type": "mistral",
    "num_hidden_layers": 32, "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 128, "intermediate_size": 14336, "vocab_size": 32000, "rope_theta": 10000.0,
    "sliding_window": 4096, "rms_norm_eps": 1e-5, "max_position_embeddings": 32768,
    "tie_word_embeddings": False, "hidden_act": "silu", "bos_token_id": 1, "eos_token_id": 2,
}
# Other sizes of the same architecture, for measurements beyond the headline (--sizes).
OTHER_SIZES = {
    "7b-v0.3": dict(MISTRAL_7B, vocab_size=32768, rope_theta=1e6, sliding_window=None),
    "nemo-12b": dict(MISTRAL_7B, num_hidden_layers=40, hidden_size=5120, vocab_size=131072, rope_theta=1e6,
                     sliding_window=None, max_position_embeddings=131072),
}
SIZE_NAMES = {"7b-v0.1": "Mistral-7B-v0.1 sizes", "7b-v0.3": "Mistral-7B-v0.3 sizes", "nemo-12b": "Mistral-NeMo-12B sizes"}
CONTEXT = 2048          # tokens each sequence holds when decoding starts
MAX_CONTEXT = 4096      # the benchmark's context length: what each sequence's cache may grow to
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            raw = json.load(f)
        out = {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]), "source": "measured"}
        if "bf16_tflops_sustained" in raw:
            out["bf16_tflops_sustained"] = float(raw["bf16_tflops_sustained"])
        return out
    except (OSError, KeyError, ValueError, TypeError):
        return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        threading.Thread(target=self._read, daemon=True).start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def mark(self):
        return len(self.rows)

    def stop(self):
        if self.proc:
            self.proc.terminate()

    def summary(self, lo=0, hi=None):
        rows = [r for r in self.rows[lo:hi] if len(r) >= 6 and r[0].isdigit()]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": statistics.median(int(r[0]) for r in rows), "sm_max_mhz": int(rows[0][1]),
                "reasons": reasons, "samples": len(rows)}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (reported)")
    ap.add_argument("--sizes", default="7b-v0.1", choices=sorted(SIZE_NAMES), help="layer sizes (default: the headline configuration)")
    ap.add_argument("--max-context", type=int, default=MAX_CONTEXT, help="what each sequence's cache may grow to")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS)
    ap.add_argument("--points", default="1,64", help="other decode batch sizes to report, comma separated ('' = none)")
    ap.add_argument("--no-prefill", action="store_true")
    ap.add_argument("--context", type=int, default=CONTEXT, help="tokens each sequence holds when decoding starts")
    a = ap.parse_args()

    if a.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust crate (no setup.py/pyproject; no cargo or rustc on this image), "
                          "pip cannot install it and it has no GPU or safetensors path"}))
        return 0
    if a.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    if a.warmup < 3:
        a.warmup = 3

    import numpy as np
    import torch
    from inference_engine_rust_b200 import LoadedModel, Sampler, SamplingParams
    from inference_engine_rust_b200.csrc import bindings as B

    pk = peaks()
    base = MISTRAL_7B if a.sizes == "7b-v0.1" else OTHER_SIZES[a.sizes]
    full_layers = base["num_hidden_layers"]
    a.layers = a.layers or full_layers
    a.max_context = max(a.max_context, a.context + 3 * (a.steps + a.warmup) + 8, a.prefill_tokens)
    cfg = dict(base, num_hidden_layers=a.layers)
    t0 = time.time()
    model = LoadedModel.random(cfg, seed=0, dtype="bfloat16", std=0.02, on_device=True)
    torch.cuda.synchronize()
    load_s = time.time() - t0
    batches = [a.batch] + [int(b) for b in a.points.split(",") if b.strip()]
    biggest = max(batches)
    per_seq = -(-(a.context + 3 * (a.steps + a.warmup) + 8) // 64) * 64     # the timed run and the two end-to-end runs
    session = model.session(max_tokens=max(biggest * per_seq, -(-a.prefill_tokens // 64) * 64), max_sequences=biggest, max_seq_len=a.max_context)
    eng = session.engine
    sampler = Sampler(SamplingParams(temperature=0.0), eng.rt.err)
    rng = np.random.default_rng(0)
    vocab = cfg["vocab_size"]
    clocks = ClockSampler()
    clocks.start()

    def prefill_slots(n):
        slots = []
        for _ in range(n):
            s = eng.open_sequence()
            eng.step([(s, rng.integers(0, vocab, a.context).tolist())], want=None)
            slots.append(s)
        torch.cuda.synchronize()
        return slots

    def decode_device(slots, steps, warmup):
        """K steps timed on the device; tokens of each step are given by the host ahead of
        time (random ids), the next-token choice is launched but not waited for."""
        n = len(slots)
        toks = rng.integers(0, vocab, (steps + warmup, n))
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches0 = 0
        for i in range(steps + warmup):
            if i == warmup:
                torch.cuda.synchronize()
                launches0 = B.launch_count + eng.graph_launches
                start.record()
            logits = eng.step([(s, [int(t)]) for s, t in zip(slots, toks[i])], want="last")
            sampler.sample_device(logits, list(range(n)), [i] * n)
        end.record()
        torch.cuda.synchronize()
        eng.check_device()
        launches = B.launch_count + eng.graph_launches - launches0
        return start.elapsed_time(end) / steps, launches

    def decode_e2e(slots, steps, warmup):
        """The same through the call a user makes every step: host ids in (pinned staging and
        one copy to the device), host ids out (the sampled tokens read back)."""
        n = len(slots)
        cur = rng.integers(0, vocab, n).tolist()
        h2d = d2h = 0
        for i in range(steps + warmup):
            if i == warmup:
                torch.cuda.synchronize()
                t_start = time.perf_counter()
                h2d = d2h = 0
            logits = eng.step([(s, [t]) for s, t in zip(slots, cur)], want="last")
            cur = sampler(logits, list(range(n)), [i] * n)
            h2d += eng.h2d_bytes_last_step
            d2h += 4 * n + 4
        torch.cuda.synchronize()
        dt = time.perf_counter() - t_start
        return dt * 1e3 / steps, h2d // steps, d2h // steps

    def decode_e2e_run_ahead(slots, steps, warmup):
        """As the library's generation loop runs it: the ids chosen on the device feed the next step
        from device memory, and the host reads every step's ids while the next step runs."""
        n = len(slots)
        reqs = list(range(n))
        logits = eng.step([(s, [int(t)]) for s, t in zip(slots, rng.integers(0, vocab, n))], want="last")
        chosen = sampler.sample_device(logits, reqs, [0] * n)
        pending = sampler.read_async(chosen)
        for i in range(steps + warmup):
            if i == warmup:
                torch.cuda.synchronize()
                t_start = time.perf_counter()
            logits = eng.step_tokens_on_device(slots, chosen)
            pending.wait()
            chosen = sampler.sample_device(logits, reqs, [i + 1] * n)
            pending = sampler.read_async(chosen)
        pending.wait()
        torch.cuda.synchronize()
        return (time.perf_counter() - t_start) * 1e3 / steps

    result = {}
    points = {}
    main_stats = None
    for nb in batches:
        slots = prefill_slots(nb)
        m0 = clocks.mark()
        ms, launches = decode_device(slots, a.steps, a.warmup)
        m1 = clocks.mark()
        if nb == a.batch and main_stats is None:
            kv_bytes = eng.cache.kv_bytes_read(slots)
            e2e_ms, h2d, d2h = decode_e2e(slots, min(a.steps, 64), a.warmup)
            ahead_ms = decode_e2e_run_ahead(slots, min(a.steps, 64), a.warmup)
            main_stats = dict(ms=ms, launches=launches, kv_bytes=kv_bytes, e2e_ms=e2e_ms, h2d=h2d, d2h=d2h, ahead_ms=ahead_ms,
                              clocks=clocks.summary(m0, m1))
        else:
            points[f"decode_b{nb}"] = round(nb * 1e3 / ms, 1)
        for s in slots:
            eng.close_sequence(s)

    prefill = None
    if not a.no_prefill:
        prompt = rng.integers(0, vocab, a.prefill_tokens).tolist()
        times = []
        for i in range(3 + 5):
            s = eng.open_sequence()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            eng.step([(s, prompt)], want="last")
            end.record()
            torch.cuda.synchronize()
            eng.close_sequence(s)
            if i >= 3:
                times.append(start.elapsed_time(end))
        pms = statistics.median(times)
        H, I, V, L = cfg["hidden_size"], cfg["intermediate_size"], vocab, a.layers
        qkv = (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * cfg["head_dim"]
        qd = cfg["num_attention_heads"] * cfg["head_dim"]
        T = a.prefill_tokens
        flops = 2 * T * L * (H * qkv + qd * H + 3 * H * I) + 2 * H * V + L * 2 * T * T * qd
        prefill = {"value": round(T * 1e3 / pms, 1), "tokens": T, "ms": round(pms, 3),
                   "frac": round(flops / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4), "unit": "tokens/s",
                   "tflops": round(flops / (pms * 1e-3) / 1e12, 1), "peak_tflops": pk["bf16_tflops"],
                   "runs": len(times), "ms_min": round(min(times), 3), "ms_max": round(max(times), 3)}
        if "bf16_tflops_sustained" in pk:      # the step is tens of milliseconds of dense tensor work
            prefill["frac_of_sustained"] = round(flops / (pms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4)
    clocks.stop()

    ms = main_stats["ms"]
    weight_bytes = model.model.weight_bytes_per_step()
    step_bytes = weight_bytes + main_stats["kv_bytes"]
    achieved = step_bytes / (ms * 1e-3) / 1e9
    value = a.batch * 1e3 / ms
    line = {
        "metric": "decode tok/s at batch 1/8/64; prefill tok/s at 2,048 tokens (Mistral 7B)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random weights N(0, 0.02), uniform random token ids)",
        "impl": "ours",
        "config": {"model": SIZE_NAMES[a.sizes], "layers": a.layers, "layers_of_config": full_layers,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": vocab, "sliding_window": cfg["sliding_window"],
                   "rope_theta": cfg["rope_theta"], "rms_norm_eps": cfg["rms_norm_eps"],
                   "global_batch": a.batch, "seq_len": a.context, "max_context": a.max_context,
                   "prefill_tokens": a.prefill_tokens, "parallelism": "single GPU",
                   "l2": "inputs larger than L2 (weights read per step exceed 126 MB many times)",
                   "peaks": pk["source"]},
        "e2e": {"value": round(a.batch * 1e3 / main_stats["e2e_ms"], 1), "unit": "tokens/s",
                "h2d_bytes_per_step": main_stats["h2d"], "d2h_bytes_per_step": main_stats["d2h"],
                # the same loop as generate() runs it: ids fed from device memory, read on the host one step behind
                "run_ahead_value": round(a.batch * 1e3 / main_stats["ahead_ms"], 1)},
        "gpu_launches": main_stats["launches"],
        "clocks": main_stats["clocks"],
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "load_s": round(load_s, 1),
    }
    if prefill:
        line["prefill"] = prefill
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
