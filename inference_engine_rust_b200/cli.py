"""Command line in the reference's manner (src/main.rs:23-50): `-m/--model`, `-n/--new-tokens`
(default 20) and a positional PROMPT, or one line on standard input when it is omitted.
The reference tokenizes text (`-t/--tokenizer`, `--chat`); tokenizers are outside this
library, so PROMPT is a list of token ids separated by spaces or commas and the
continuation is printed as ids.  Generation stops at the configuration's EOS id
(src/main.rs:100) unless `--stop-token` says otherwise (the reference's chat front-end has
the same option, src/bin/chat.rs:49-51).

    python -m inference_engine_rust_b200 -m DIR -n 32 "1 415 7 88"
    python -m inference_engine_rust_b200 random-model --config config.json --seed 0 --out DIR
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


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "random-model":
        return _random_model(argv[1:])
    ap = argparse.ArgumentParser(prog="inference_engine_rust_b200",
                                 description="Greedy or sampled generation from a model folder (token ids in, token ids out)")
    ap.add_argument("-m", "--model", default="model/mistral-7b-v0.1",
                    help="model folder with config.json and safetensors (relative to cwd is fine)")
    ap.add_argument("-n", "--new-tokens", type=int, default=20, help="how many new tokens to append after the prompt")
    ap.add_argument("--temperature", type=float, default=0.0, help="0 = greedy; > 0 = temperature sampling")
    ap.add_argument("--seed", type=int, default=0, help="seed of the sampling draws")
    ap.add_argument("--stop-token", type=int, action="append", default=None,
                    help="stop id (repeatable); default: the configuration's EOS; a negative id = never stop")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--max-tokens", type=int, default=None, help="positions the cache holds (default: prompt + new tokens)")
    ap.add_argument("--plain", action="store_true", help="run the plain reference kernels only")
    ap.add_argument("prompt", nargs="?", metavar="PROMPT", help="token ids; if omitted, one line is read from stdin")
    a = ap.parse_args(argv)

    if a.prompt is not None:
        if not a.prompt.strip():
            print("error: prompt is empty", file=sys.stderr)                 # src/main.rs:59-61
            return 2
        text = a.prompt
    else:
        text = sys.stdin.readline().rstrip("\r\n")
    if not text.strip():
        print("error: no prompt: pass PROMPT or pipe a line on stdin", file=sys.stderr)   # src/main.rs:71-75
        return 2
    try:
        ids = parse_ids(text)
    except ValueError as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
    if a.new_tokens < 0:
        print("error: --new-tokens must be >= 0", file=sys.stderr)
        return 2

    from .api import LoadedModel
    model = LoadedModel.load(a.model, dtype=a.dtype, plain_kernels=a.plain)
    max_tokens = a.max_tokens or (len(ids) + a.new_tokens + 64)
    session = model.session(max_tokens=max_tokens)
    stop = None if a.stop_token is None else [s for s in a.stop_token if s >= 0]
    out = session.generate([ids], max_new_tokens=a.new_tokens, temperature=a.temperature, seed=a.seed,
                           stop_ids=stop)[0]
    print(" ".join(str(t) for t in out))
    return 0
