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

# Layer sizes come from the package's named configurations (the library itself takes every size
# from config.json): Mistral 7B v0.1 is the benchmark configuration, the other two are measured
# beside it (`points`) and on their own (--sizes).
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


class Rig:
    """One random-weight model of a named configuration with a session sized for the batches to be
    measured, and the measurements themselves."""

    def __init__(self, sizes: str, layers, batches, context: int, max_context: int, prefill_tokens: int,
                 steps: int, warmup: int, seed: int = 0):
        import numpy as np
        import torch
        from inference_engine_rust_b200 import LoadedModel, Sampler, SamplingParams
        from inference_engine_rust_b200.config import preset
        self.np, self.torch = np, torch
        base = preset(sizes)
        self.full_layers = base["num_hidden_layers"]
        self.layers = layers or self.full_layers
        self.cfg = dict(base, num_hidden_layers=self.layers)
        self.context, self.prefill_tokens = context, prefill_tokens
        self.max_context = max(max_context, context + 3 * (steps + warmup) + 8, prefill_tokens)
        t0 = time.time()
        self.model = LoadedModel.random(self.cfg, seed=seed, dtype="bfloat16", std=0.02, on_device=True)
        torch.cuda.synchronize()
        self.load_s = time.time() - t0
        biggest = max(batches)
        per_seq = -(-(context + 3 * (steps + warmup) + 8) // 64) * 64     # the timed run and the two end-to-end runs
        self.session = self.model.session(max_tokens=max(biggest * per_seq, -(-prefill_tokens // 64) * 64),
                                          max_sequences=biggest, max_seq_len=self.max_context)
        self.eng = self.session.engine
        self.sampler = Sampler(SamplingParams(temperature=0.0), self.eng.rt.err)
        self.rng = np.random.default_rng(0)
        self.vocab = self.cfg["vocab_size"]

    def close(self):
        self.model = self.session = self.eng = self.sampler = None
        self.torch.cuda.empty_cache()

    def prefill_slots(self, n):
        slots = []
        for _ in range(n):
            s = self.eng.open_sequence()
            self.eng.step([(s, self.rng.integers(0, self.vocab, self.context).tolist())], want=None)
            slots.append(s)
        self.torch.cuda.synchronize()
        return slots

    def release(self, slots):
        for s in slots:
            self.eng.close_sequence(s)

    def decode_device(self, slots, steps, warmup):
        """K steps timed on the device; tokens of each step are given by the host ahead of
        time (random ids), the next-token choice is launched but not waited for."""
        from inference_engine_rust_b200.csrc import bindings as B
        torch, eng = self.torch, self.eng
        n = len(slots)
        toks = self.rng.integers(0, self.vocab, (steps + warmup, n))
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches0 = 0
        for i in range(steps + warmup):
            if i == warmup:
                torch.cuda.synchronize()
                launches0 = B.launch_count + eng.graph_launches
                start.record()
            logits = eng.step([(s, [int(t)]) for s, t in zip(slots, toks[i])], want="last")
            self.sampler.sample_device(logits, list(range(n)), [i] * n)
        end.record()
        torch.cuda.synchronize()
        eng.check_device()
        launches = B.launch_count + eng.graph_launches - launches0
        return start.elapsed_time(end) / steps, launches

    def decode_e2e(self, slots, steps, warmup):
        """The same through the call a user makes every step: host ids in (pinned staging and
        one copy to the device), host ids out (the sampled tokens read back)."""
        torch, eng = self.torch, self.eng
        n = len(slots)
        cur = self.rng.integers(0, self.vocab, n).tolist()
        h2d = d2h = 0
        for i in range(steps + warmup):
            if i == warmup:
                torch.cuda.synchronize()
                t_start = time.perf_counter()
                h2d = d2h = 0
            logits = eng.step([(s, [t]) for s, t in zip(slots, cur)], want="last")
            cur = self.sampler(logits, list(range(n)), [i] * n)
            h2d += eng.h2d_bytes_last_step
            d2h += 4 * n + 4
        torch.cuda.synchronize()
        dt = time.perf_counter() - t_start
        return dt * 1e3 / steps, h2d // steps, d2h // steps

    def decode_e2e_run_ahead(self, slots, steps, warmup):
        """As the library's generation loop runs it: the ids chosen on the device feed the next step
        from device memory, and the host reads every step's ids while the next step runs."""
        torch, eng, sampler = self.torch, self.eng, self.sampler
        n = len(slots)
        reqs = list(range(n))
        logits = eng.step([(s, [int(t)]) for s, t in zip(slots, self.rng.integers(0, self.vocab, n))], want="last")
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

    def step_bytes(self, slots):
        """Bytes a one-token step over `slots` has to read: every weight once, the live keys and values."""
        return self.model.model.weight_bytes_per_step() + self.eng.cache.kv_bytes_read(slots)

    def prefill_flops(self):
        cfg, T, L = self.cfg, self.prefill_tokens, self.layers
        H, I, V = cfg["hidden_size"], cfg["intermediate_size"], self.vocab
        qkv = (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * cfg["head_dim"]
        qd = cfg["num_attention_heads"] * cfg["head_dim"]
        return 2 * T * L * (H * qkv + qd * H + 3 * H * I) + 2 * H * V + L * 2 * T * T * qd

    def prefill(self, runs=5, warm=3, idle_s=0.0):
        """Device times of whole-prompt steps, one after another; with `idle_s` the device rests that long
        before each timed step (a step that starts below the power cap, as a prompt between one-token
        steps does, against steps back to back, which settle at the cap)."""
        torch, eng = self.torch, self.eng
        prompt = self.rng.integers(0, self.vocab, self.prefill_tokens).tolist()
        times = []
        for i in range(warm + runs):
            if idle_s and i >= warm:
                torch.cuda.synchronize()
                time.sleep(idle_s)
            s = eng.open_sequence()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            eng.step([(s, prompt)], want="last")
            end.record()
            torch.cuda.synchronize()
            eng.close_sequence(s)
            if i >= warm:
                times.append(start.elapsed_time(end))
        return times

    # ---- where a layer's time goes inside the replayed graph --------------------------------------
    def timeline(self, batch: int):
        """Medians of the projection kernels' time stamps (device-wide timer) over the CTAs of each launch of
        the last replayed one-token step.  Needs a build that records them: IERT_EXTRA_DEFINES=IERT_GEMM_TRACE."""
        import ctypes
        import numpy as np
        from inference_engine_rust_b200.csrc import bindings as B
        lib = B.core()
        if not hasattr(lib, "iert_gemm_tc_trace_read"):
            return None
        slots = self.prefill_slots(batch)
        self.decode_device(slots, 6, 3)
        self.torch.cuda.synchronize()
        launches = []
        names = {"tc": ["start", "weights asked", "dependency", "operands", "last MMA", "accumulator", "partial out", "end"],
                 "rows": ["start", "weights asked", "dependency", "last stage asked", "first stage full", "last stage full", "", "end"]}
        for kind, fn, ctas in (("tc", "iert_gemm_tc_trace_read", 304), ("rows", "iert_gemm_rows_trace_read", 512)):
            stamps = np.zeros((64, ctas, 8), dtype=np.uint64)
            meta = np.zeros((64, 8), dtype=np.int32)
            f = getattr(lib, fn)
            f.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
            if f(stamps.ctypes.data, meta.ctypes.data) != 0:
                return None
            for i in range(64):
                if meta[i, 2] > 0:
                    st = stamps[i, :min(int(meta[i, 4]), ctas)].astype(np.int64)
                    if (st[:, 0] > 0).any():
                        launches.append((kind, meta[i].tolist(), st))
        launches.sort(key=lambda e: np.median(e[2][:, 0][e[2][:, 0] > 0]))
        launches = launches[-(4 * self.layers + 1):]              # the last step's projections and its output head
        t0 = min(int(e[2][e[2] > 0].min()) for e in launches)
        out = []
        for kind, meta, st in launches:
            row = {"kernel": "gemm_tc" if kind == "tc" else "gemm_rows", "tokens": meta[1], "rows": meta[2], "k": meta[3],
                   "ctas": meta[4], "us": {}}
            for c, name in enumerate(names[kind]):
                col = st[:, c]
                col = col[col > 0]
                if name and len(col):
                    row["us"][name] = round((float(np.median(col)) - t0) / 1e3, 2)
            row["us"]["last CTA's end"] = round((int(st.max()) - t0) / 1e3, 2)
            out.append(row)
        self.release(slots)
        return out

    # ---- the dominant kernels one by one -----------------------------------------------------
    def kernel_table(self, batch: int, pk):
        """CUDA-event times of the projections (at `batch` tokens and at the prefill length) and of
        decode attention (over the live cache of `batch` sequences), each launched once per layer
        in turn so that its operands come from memory, not from the L2 (32 layers of weights)."""
        import torch
        from inference_engine_rust_b200.parts.base import StepContext
        from inference_engine_rust_b200.csrc import bindings as B
        eng, rt, cfg = self.eng, self.eng.rt, self.cfg
        blocks = eng.model.blocks
        H, I = cfg["hidden_size"], cfg["intermediate_size"]
        stream = B.stream_ptr()
        out = []

        def timed(fn, reps):
            for _ in range(2):
                fn()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            for _ in range(reps):
                fn()
            end.record()
            torch.cuda.synchronize()
            return start.elapsed_time(end) * 1e3 / (reps * len(blocks))          # us per launch

        for M, what in ((batch, f"one-token step, {batch} tokens"), (self.prefill_tokens, f"prompt, {self.prefill_tokens} tokens")):
            x = (torch.randn(M, H, device=rt.device) * 0.5).bfloat16()
            a_in = (torch.randn(M, I, device=rt.device) * 0.5).bfloat16()
            res = torch.zeros(M, H, device=rt.device)
            q_out = torch.empty(M, blocks[0].mixer.qkv.out_features, device=rt.device, dtype=torch.bfloat16)
            act = torch.empty(M, I, device=rt.device, dtype=torch.bfloat16)
            o_in = (torch.randn(M, blocks[0].mixer.q_dim, device=rt.device) * 0.5).bfloat16()
            from inference_engine_rust_b200.parts import fast_linear
            cases = [
                ("qkv", lambda b: b.mixer.qkv.apply(x, q_out, M, stream), blocks[0].mixer.qkv),
                ("o + residual", lambda b: b.mixer.o.apply(o_in, res, M, stream, add_residual=True), blocks[0].mixer.o),
                ("gate-up + silu", lambda b: fast_linear.apply_gated(b.ffn.gate_up, x, act, M, stream), blocks[0].ffn.gate_up),
                ("down + residual", lambda b: b.ffn.down.apply(a_in, res, M, stream, add_residual=True), blocks[0].ffn.down),
            ]
            for name, call, lin in cases:
                us = timed(lambda: [call(b) for b in blocks], 3)
                n, k = lin.weight.shape
                flops, nbytes = 2.0 * M * n * k, lin.nbytes()
                row = {"kernel": name, "where": what, "us": round(us, 2)}
                if M <= 64:
                    row["gb_s"] = round(nbytes / us / 1e3, 1)
                    row["frac"] = round(nbytes / us / 1e3 / pk["hbm_gbs"], 3)
                else:
                    row["tflops"] = round(flops / us / 1e6, 1)
                    row["frac"] = round(flops / us / 1e6 / pk["bf16_tflops"], 3)
                out.append(row)
        # decode attention over the live cache: the mixer's own kernel, layer after layer
        slots = self.prefill_slots(batch)
        n = len(slots)
        o_cu, o_slot, o_pos, o_seq, o_tok, o_rows, total = eng._layout(n, n, 0)
        meta = torch.zeros(total, dtype=torch.int32, device=rt.device)
        pos0 = [eng.length(s) for s in slots]
        meta[o_cu:o_cu + n + 1] = torch.arange(n + 1, dtype=torch.int32)
        meta[o_slot:o_slot + n] = torch.tensor(slots, dtype=torch.int32)
        meta[o_pos:o_pos + n] = torch.tensor(pos0, dtype=torch.int32)
        meta[o_seq:o_seq + n] = torch.arange(n, dtype=torch.int32)
        for s in slots:
            eng.cache.reserve(s, eng.length(s) + 1)
        eng.cache.upload()
        ctx = eng._context("decode", meta, n, n, [1] * n, pos0, slots)
        from inference_engine_rust_b200.parts import fast_attention
        mix = blocks[0].mixer
        qkv = (torch.randn(n, mix.q_dim + 2 * mix.kv_dim, device=rt.device) * 0.5).bfloat16()
        a_out = torch.empty(n, mix.q_dim, device=rt.device, dtype=torch.bfloat16)
        views = [eng.cache.layer_view(eng.model.spec.cache_entry(i)) for i in range(len(blocks))]
        us = timed(lambda: [fast_attention.decode_with_rotation(b.mixer, qkv, a_out, ctx, v, True) for b, v in zip(blocks, views)], 3)
        kv_bytes = eng.cache.kv_bytes_read(slots) / len(blocks)
        out.append({"kernel": "decode attention (rotation, cache write, merge of the splits)", "where": f"{batch} sequences of {self.context} tokens",
                    "us": round(us, 2), "gb_s": round(kv_bytes / us / 1e3, 1), "frac": round(kv_bytes / us / 1e3 / pk["hbm_gbs"], 3)})
        eng.check_device()
        self.release(slots)
        # prompt attention over one prompt of the prefill length (the kernel alone: queries, keys and values
        # of one layer from a random projection, a fresh buffer per launch so that nothing waits in the L2)
        import numpy as np
        T, W = self.prefill_tokens, mix.q_dim + 2 * mix.kv_dim
        if T >= 2:
            reps = max(2, min(8, int(400e6 // (T * W * 2)) + 1))
            bufs = [(torch.randn(T, W, device=rt.device) * 0.7).bfloat16() for _ in range(reps)]
            p_out = torch.empty(T, mix.q_dim, device=rt.device, dtype=torch.bfloat16)
            arrs = [torch.tensor(a, dtype=torch.int32, device=rt.device) for a in ([0, T], [0], np.zeros(T, dtype=np.int32), [0])]
            view = B.BatchView(cu_q=arrs[0].data_ptr(), slot_ids=arrs[1].data_ptr(), tok_seq=arrs[2].data_ptr(),
                               pos0=arrs[3].data_ptr(), n_seqs=1, n_tokens=T)
            turn = [0]

            def one():
                turn[0] += 1
                assert B.attention_prefill(bufs[turn[0] % reps], p_out, view, mix.heads, mix.kv_heads, mix.head_dim,
                                           mix.window or 0, mix.scale, T, stream, err=rt.err)
            for _ in range(3):
                one()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            for _ in range(2 * reps):
                one()
            end.record()
            torch.cuda.synchronize()
            us = start.elapsed_time(end) * 1e3 / (2 * reps)
            window = mix.window or T
            flops = 4.0 * mix.head_dim * mix.heads * sum(min(i + 1, window) for i in range(T))
            out.append({"kernel": "prompt attention", "where": f"one prompt of {T} tokens", "us": round(us, 2),
                        "tflops": round(flops / us / 1e6, 1), "frac": round(flops / us / 1e6 / pk["bf16_tflops"], 3)})
            eng.check_device()
        return out


def other_sizes_points(pk, steps: int, warmup: int):
    """Short measurements at the two other configurations of the architecture: Mistral 7B v0.3 sizes
    with eight sequences at 8,192 tokens of context, Mistral NeMo 12B sizes at batch 32 and batch 1
    (2,048 tokens of context) and its 2,048-token prefill.  Each with its fraction of the measured
    peak (the one-token steps of the memory rate, the prefill of the tensor rate)."""
    pts = {}
    rig = Rig("7b-v0.3", None, [8], 8192, 16384, 64, steps, warmup, seed=1)
    slots = rig.prefill_slots(8)
    ms, _ = rig.decode_device(slots, steps, warmup)
    pts["v03_b8_ctx8192_ms"] = round(ms, 3)
    pts["v03_b8_ctx8192_frac"] = round(rig.step_bytes(slots) / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
    rig.release(slots)
    rig.close()
    rig = Rig("nemo-12b", None, [32, 1], 2048, 4096, 2048, steps, warmup, seed=2)
    for nb, key in ((32, "nemo_b32"), (1, "nemo_b1")):
        slots = rig.prefill_slots(nb)
        ms, _ = rig.decode_device(slots, steps, warmup)
        if nb == 1:
            pts["nemo_b1_tok_s"] = round(1e3 / ms, 1)
        else:
            pts["nemo_b32_ms"] = round(ms, 3)
        pts[key + "_frac"] = round(rig.step_bytes(slots) / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        rig.release(slots)
    times = rig.prefill(runs=3, warm=2)
    pms = statistics.median(times)
    pts["nemo_prefill_2048_ms"] = round(pms, 2)
    pts["nemo_prefill_2048_frac"] = round(rig.prefill_flops() / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)
    rig.close()
    return pts


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
    ap.add_argument("--no-other-sizes", action="store_true",
                    help="skip the short measurements at Mistral 7B v0.3 and NeMo 12B sizes (points v03_*, nemo_*)")
    ap.add_argument("--timeline", action="store_true",
                    help="print, instead of the benchmark line, when the CTAs of each projection launch of a replayed "
                         "one-token step passed their marked points (us, medians per launch); needs "
                         "IERT_EXTRA_DEFINES=IERT_GEMM_TRACE in the environment, and --layers of 2 or 3")
    ap.add_argument("--kernels", action="store_true",
                    help="also time the dominant kernels one by one with CUDA events (projections and decode "
                         "attention at the decode batch, projections at the prefill length): key 'kernels'")
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

    pk = peaks()
    if a.timeline:
        rig = Rig(a.sizes, a.layers or 3, [a.batch], a.context, a.max_context, a.prefill_tokens, a.steps, a.warmup)
        rows = rig.timeline(a.batch)
        rig.close()
        if rows is None:
            print("bench.py --timeline: the kernels were built without IERT_EXTRA_DEFINES=IERT_GEMM_TRACE")
            return 2
        for r in rows:
            print(json.dumps(r))
        return 0
    batches = [a.batch] + [int(b) for b in a.points.split(",") if b.strip()]
    rig = Rig(a.sizes, a.layers, batches, a.context, a.max_context, a.prefill_tokens, a.steps, a.warmup)
    cfg, vocab = rig.cfg, rig.vocab
    clocks = ClockSampler()
    clocks.start()

    points = {}
    main_stats = None
    for nb in batches:
        slots = rig.prefill_slots(nb)
        m0 = clocks.mark()
        ms, launches = rig.decode_device(slots, a.steps, a.warmup)
        m1 = clocks.mark()
        if nb == a.batch and main_stats is None:
            step_bytes = rig.step_bytes(slots)
            e2e_ms, h2d, d2h = rig.decode_e2e(slots, min(a.steps, 64), a.warmup)
            ahead_ms = rig.decode_e2e_run_ahead(slots, min(a.steps, 64), a.warmup)
            main_stats = dict(ms=ms, launches=launches, step_bytes=step_bytes, e2e_ms=e2e_ms, h2d=h2d, d2h=d2h,
                              ahead_ms=ahead_ms, clocks=clocks.summary(m0, m1))
        else:
            points[f"decode_b{nb}"] = round(nb * 1e3 / ms, 1)
            points[f"decode_b{nb}_frac"] = round(rig.step_bytes(slots) / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        rig.release(slots)

    prefill = None
    if not a.no_prefill:
        times = rig.prefill()
        pms = statistics.median(times)
        T, flops = a.prefill_tokens, rig.prefill_flops()
        prefill = {"value": round(T * 1e3 / pms, 1), "tokens": T, "ms": round(pms, 3),
                   "frac": round(flops / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4), "unit": "tokens/s",
                   "tflops": round(flops / (pms * 1e-3) / 1e12, 1), "peak_tflops": pk["bf16_tflops"],
                   "runs": len(times), "ms_min": round(min(times), 3), "ms_max": round(max(times), 3)}
        if "bf16_tflops_sustained" in pk:      # the step is tens of milliseconds of dense tensor work
            prefill["frac_of_sustained"] = round(flops / (pms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4)
        # The steps above run back to back and settle at the power cap, as the sustained peak does.  The burst
        # peak is a kernel that starts below the cap; its counterpart is a step after a second of rest.
        rested = rig.prefill(runs=3, warm=0, idle_s=1.0)
        rms = statistics.median(rested)
        prefill.update({"ms_after_1s_idle": round(rms, 3), "ms_after_1s_idle_min": round(min(rested), 3),
                        "ms_after_1s_idle_max": round(max(rested), 3),
                        "frac_after_1s_idle": round(flops / (rms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                        "runs_after_1s_idle": len(rested)})
    kernels = rig.kernel_table(a.batch, pk) if a.kernels else None
    load_s, layers, full_layers, max_context = rig.load_s, rig.layers, rig.full_layers, rig.max_context
    rig.close()
    if not a.no_other_sizes and a.sizes == "7b-v0.1" and a.layers is None:
        points.update(other_sizes_points(pk, min(a.steps, 32), max(3, min(a.warmup, 4))))
    clocks.stop()

    ms = main_stats["ms"]
    achieved = main_stats["step_bytes"] / (ms * 1e-3) / 1e9
    value = a.batch * 1e3 / ms
    line = {
        "metric": "decode tok/s at batch 1/8/64; prefill tok/s at 2,048 tokens (Mistral 7B)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random weights N(0, 0.02), uniform random token ids)",
        "impl": "ours",
        "config": {"model": SIZE_NAMES[a.sizes], "layers": layers, "layers_of_config": full_layers,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": vocab, "sliding_window": cfg["sliding_window"],
                   "rope_theta": cfg["rope_theta"], "rms_norm_eps": cfg["rms_norm_eps"],
                   "global_batch": a.batch, "seq_len": a.context, "max_context": max_context,
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
    if kernels is not None:
        line["kernels"] = kernels
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
