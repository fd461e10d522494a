"""Command line in the reference's manner (src/main.rs:23-50): `-m/--model`, `-n/--new-tokens`
(default 20) and a positional PROMPT, or one line on standard input when it is omitted.
The reference tokenizes text (`-t/--tokenizer`, `--chat`); tokenizers are outside this
library, so PROMPT is a list of token ids separated by spaces or commas and the
continuation is printed as ids.  Generation stops at the configuration's EOS id
(src/main.rs:100) unless `--stop-token` says otherwise (the reference's chat front-end has
the same option, src/bin/chat.rs:49-51).

    python -m inference_engine_rust_b200 -m DIR -n 32 "1 415 7 88"
    python -m inference_engine_rust_b200 -m DIR -n 32 --prompt-file requests.txt     # one request per line, run as batches
    python -m inference_engine_rust_b200 --random tiny-a --seed 3 -n 8 "1 5 9"       # no folder: seeded random weights
    python -m inference_engine_rust_b200 random-model --config config.json --seed 0 --out DIR
    python -m inference_engine_rust_b200 bench -m DIR [--json] [--runs 5] all --decode-tokens 128

`bench` is the reference's bench_compare (src/bin/bench_compare.rs:30-87): the subcommands
`all`, `cold-start`, `interactive-ttft` and `decode-throughput -n N`, with `-p/--prompt`,
`--json`, `--min-decode-tps` and `--runs` (at least 5).
"""
from __future__ import annotations

import argparse
import json
import re
import sys
from typing import List, Optional


def parse_ids(text: str) -> List[int]:
    parts = [p for p in re.split(r"[\s,]+", text.strip()) if p]
    try:
        return [int(p) for p in parts]
    except ValueError:
        raise ValueError(f"the prompt must be token ids separated by spaces or commas, got {text!r}") from None


def _random_model(argv: List[str]) -> int:
    ap = argparse.ArgumentParser(prog="inference_engine_rust_b200 random-model",
                                 description="Write a model folder (config.json, model.safetensors) with seeded random weights")
    ap.add_argument("--config", required=True, help="a config.json to take the sizes from")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"], help="storage type of the tensors")
    ap.add_argument("--std", type=float, default=0.02, help="standard deviation of the normal weights")
    ap.add_argument("--out", required=True, help="folder to write")
    a = ap.parse_args(argv)
    from .api import write_random_model
    with open(a.config, "r", encoding="utf-8") as f:
        raw = json.load(f)
    write_random_model(a.out, raw, seed=a.seed, dtype=a.dtype, std=a.std)
    print(a.out)
    return 0


def _bench(argv: List[str]) -> int:
    from . import bench_metrics as M
    ap = argparse.ArgumentParser(prog="inference_engine_rust_b200 bench",
                                 description="Latency/throughput metrics of a model folder (cold TTFT, interactive TTFT, decode tok/s)")
    ap.add_argument("-m", "--model", default="model/mistral-7b-v0.1", help="model folder")
    ap.add_argument("-p", "--prompt", default=" ".join(str(t) for t in M.DEFAULT_BENCH_PROMPT), help="prompt as token ids")
    ap.add_argument("--json", action="store_true", help="emit one JSON object")
    ap.add_argument("--min-decode-tps", type=float, default=None,
                    help="fail if measured decode tok/s is strictly below this (decode-throughput / all only)")
    ap.add_argument("--runs", type=int, default=5, help="repetitions per command (minimum 5)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--batch", type=int, default=1, help="sequences decoding together (the prompt is repeated)")
    sub = ap.add_subparsers(dest="command", required=True)
    p_all = sub.add_parser("all", help="cold start + interactive TTFT + decode throughput (single process)")
    p_all.add_argument("--decode-tokens", type=int, default=128)
    sub.add_parser("cold-start", help="from the folder on disk through the first greedy token id")
    sub.add_parser("interactive-ttft", help="weights loaded, fresh cache: prompt evaluation + first token")
    p_dec = sub.add_parser("decode-throughput", help="after a warm prefill, time greedy decode only")
    p_dec.add_argument("-n", "--decode-tokens", type=int, default=128)
    a = ap.parse_args(argv)
    if a.runs < 5:
        print("error: --runs must be at least 5 for stable comparisons", file=sys.stderr)   # bench_compare.rs:304-308
        return 2
    try:
        prompt = parse_ids(a.prompt)
    except ValueError as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
    if not prompt:
        print("error: prompt is empty", file=sys.stderr)
        return 2

    def show(title, m):
        print(f"=== {title} ===")
        for k, v in m.items():
            print(f"  {k + ':':26s}{v:.3f}" if isinstance(v, float) else f"  {k + ':':26s}{v}")

    head = {"model": a.model, "prompt": prompt, "dtype": a.dtype}
    try:
        if a.command == "all":
            runs = []
            for _ in range(a.runs):
                m = M.run_all(a.model, prompt, a.decode_tokens, dtype=a.dtype, batch=a.batch)
                M.check_decode(m["decode"], a.min_decode_tps)
                runs.append(m)
            summary = {"interactive": M.summarize_interactive([r["interactive"] for r in runs]),
                       "decode": M.summarize_decode([r["decode"] for r in runs])}
            if a.json:
                print(json.dumps({"suite": "all", **head,
                                  "runs": {k: [r[k] for r in runs] for k in ("cold", "interactive", "decode")},
                                  "summary": summary}))
            else:
                show("cold-start", runs[0]["cold"])
                show("interactive-ttft (warm weights, fresh cache)", runs[0]["interactive"])
                show("decode-throughput", runs[0]["decode"])
                print(f"=== summary over {a.runs} runs ===")
                print(f"  interactive: {json.dumps(summary['interactive'])}")
                print(f"  decode:      {json.dumps(summary['decode'])}")
        elif a.command == "cold-start":
            if a.min_decode_tps is not None:
                print("warning: --min-decode-tps ignored for cold-start", file=sys.stderr)
            runs = [M.run_cold_start(a.model, prompt, dtype=a.dtype, batch=a.batch)[0] for _ in range(a.runs)]
            if a.json:
                print(json.dumps({"suite": "cold-start", **head, "runs": runs}))
            else:
                show("cold-start", runs[0])
                print(f"  (showing run 1 of {a.runs}; use --json for all runs)")
        else:
            bench = M.EngineBench.load(a.model, dtype=a.dtype, batch=a.batch)
            if a.command == "interactive-ttft":
                runs = [bench.run_interactive_ttft(prompt) for _ in range(a.runs)]
                summary = M.summarize_interactive(runs)
                title = "interactive-ttft (warm weights, fresh cache)"
            else:
                runs = []
                for _ in range(a.runs):
                    m = bench.run_decode_throughput(prompt, a.decode_tokens)
                    M.check_decode(m, a.min_decode_tps)
                    runs.append(m)
                summary = M.summarize_decode(runs)
                title = "decode-throughput"
            if a.json:
                print(json.dumps({"suite": a.command, **head, "runs": runs, "summary": summary}))
            else:
                show(title, runs[0])
                print(f"=== summary over {a.runs} runs ===")
                print(f"  {json.dumps(summary)}")
    except (RuntimeError, ValueError, OSError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 1
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "random-model":
        return _random_model(argv[1:])
    if argv and argv[0] == "bench":
        return _bench(argv[1:])
    from .config.presets import PRESETS
    ap = argparse.ArgumentParser(prog="inference_engine_rust_b200",
                                 description="Greedy or sampled generation from a model folder (token ids in, token ids out)")
    ap.add_argument("-m", "--model", default=None,
                    help="model folder with config.json and safetensors (relative to cwd is fine; "
                         "default: model/mistral-7b-v0.1 unless --random is given)")
    ap.add_argument("--random", choices=sorted(PRESETS), default=None, metavar="PRESET",
                    help="no folder: seeded random weights for a named configuration "
                         f"({', '.join(sorted(PRESETS))}); --seed seeds them")
    ap.add_argument("-n", "--new-tokens", type=int, default=20, help="how many new tokens to append after the prompt")
    ap.add_argument("--temperature", type=float, default=0.0, help="0 = greedy; > 0 = temperature sampling")
    ap.add_argument("--seed", type=int, default=0, help="seed of the sampling draws (and of --random weights)")
    ap.add_argument("--stop-token", type=int, action="append", default=None,
                    help="stop id (repeatable); default: the configuration's EOS; a negative id = never stop")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "bf16", "float32", "fp32"])
    ap.add_argument("--max-tokens", type=int, default=None,
                    help="positions the cache holds over all requests (default: what the requests need)")
    ap.add_argument("--max-context", type=int, default=None,
                    help="the longest a single sequence may grow (default: the configuration's limit)")
    ap.add_argument("--max-batch", type=int, default=None, help="most requests that run together")
    ap.add_argument("--plain", action="store_true", help="run the plain reference kernels only")
    ap.add_argument("--ignore-extra-tensors", action="store_true",
                    help="accept a folder that carries tensors the model does not use")
    ap.add_argument("--prompt-file", default=None, metavar="FILE",
                    help="one request per line (token ids; empty lines and lines starting with # are skipped; "
                         "'-' = standard input): requests of unequal lengths run together as batches, "
                         "one output line per request")
    ap.add_argument("prompt", nargs="?", metavar="PROMPT", help="token ids; if omitted, one line is read from stdin")
    a = ap.parse_args(argv)

    if a.model is not None and a.random is not None:
        print("error: give either --model or --random, not both", file=sys.stderr)
        return 2
    if a.prompt_file is not None and a.prompt is not None:
        print("error: give either PROMPT or --prompt-file, not both", file=sys.stderr)
        return 2
    texts: List[str]
    if a.prompt_file is not None:
        try:
            f = sys.stdin if a.prompt_file == "-" else open(a.prompt_file, "r", encoding="utf-8")
        except OSError as e:
            print(f"error: {e}", file=sys.stderr)
            return 2
        with f:
            texts = [ln.strip() for ln in f if ln.strip() and not ln.lstrip().startswith("#")]
        if not texts:
            print(f"error: no request in {a.prompt_file}", file=sys.stderr)
            return 2
    elif a.prompt is not None:
        if not a.prompt.strip():
            print("error: prompt is empty", file=sys.stderr)                 # src/main.rs:59-61
            return 2
        texts = [a.prompt]
    else:
        texts = [sys.stdin.readline().rstrip("\r\n")]
        if not texts[0].strip():
            print("error: no prompt: pass PROMPT or pipe a line on stdin", file=sys.stderr)   # src/main.rs:71-75
            return 2
    try:
        requests = [parse_ids(t) for t in texts]
    except ValueError as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
    if a.new_tokens < 0:
        print("error: --new-tokens must be >= 0", file=sys.stderr)
        return 2

    from .api import LoadedModel
    from .weights import WeightError
    from .config import ConfigError
    try:
        if a.random is not None:
            from .config.presets import preset
            model = LoadedModel.random(preset(a.random), seed=a.seed, dtype=a.dtype, plain_kernels=a.plain,
                                       on_device=True)
        else:
            model = LoadedModel.load(a.model or "model/mistral-7b-v0.1", dtype=a.dtype, plain_kernels=a.plain,
                                     strict=not a.ignore_extra_tensors)
    except (WeightError, ConfigError, OSError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 1
    for note in model.model.notes:
        print(f"note: {note}", file=sys.stderr)
    limit = model.spec.max_position if a.max_context is None else min(a.max_context, model.spec.max_position)
    if limit <= 0:
        print("error: --max-context must be positive", file=sys.stderr)
        return 2
    # room for every request at its longest, each rounded up to a page, unless told otherwise
    from .cache import PAGE_TOKENS
    need = sum(-(-min(len(r) + a.new_tokens, limit) // PAGE_TOKENS) * PAGE_TOKENS for r in requests)
    session = model.session(max_tokens=a.max_tokens or need, max_seq_len=limit)
    stop = None if a.stop_token is None else [s for s in a.stop_token if s >= 0]
    try:
        outs = session.generate(requests, max_new_tokens=a.new_tokens, temperature=a.temperature, seed=a.seed,
                                stop_ids=stop, max_batch=a.max_batch)
    except ValueError as e:                      # a request that cannot fit, an id outside the vocabulary
        print(f"error: {e}", file=sys.stderr)
        return 1
    for out in outs:
        print(" ".join(str(t) for t in out))
    return 0
