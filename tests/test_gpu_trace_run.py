"""bin/trace_run as a user drives it: the same requests replayed whole, with the last 32
tokens one by one, and in batches of unequal lengths through few slots; in 32-bit and in
bfloat16; every wanted row compared with the plain implementation."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers import TINY, compare, make_folder, plain_weights, prompts_for
from plain import mistral_plain as P

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


def replay(folder, dtype, steps, out_dir, max_tokens):
    """Feed the steps line by line, waiting for `done <step>` after each."""
    proc = subprocess.Popen([sys.executable, TRACE_RUN, "--model", folder, "--dtype", dtype, "--out", out_dir,
                             "--max-tokens", str(max_tokens)],
                            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    try:
        for rec in steps:
            proc.stdin.write(json.dumps(rec) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {rec['step']}", f"expected 'done {rec['step']}', got {line!r}"
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()


def read(out_dir, step, vocab):
    return torch.from_numpy(np.fromfile(os.path.join(out_dir, f"{step}.f32"), dtype="<f4").reshape(-1, vocab))


def whole_trace(prompts):
    return [{"step": i, "entries": [{"id": f"r{i}", "tokens": p, "want": list(range(len(p)))}], "end": [f"r{i}"]}
            for i, p in enumerate(prompts)]


def tail_trace(prompts, tail=32):
    steps, where = [], {}
    for i, p in enumerate(prompts):
        t = min(tail, len(p) - 1)
        head = len(p) - t
        where[i] = [len(steps)]
        steps.append({"step": len(steps), "entries": [{"id": f"r{i}", "tokens": p[:head], "want": list(range(head))}], "end": []})
        for k in range(t):
            where[i].append(len(steps))
            steps.append({"step": len(steps), "entries": [{"id": f"r{i}", "tokens": [p[head + k]], "want": [0]}],
                          "end": [f"r{i}"] if k == t - 1 else []})
        if t == 0:
            steps[-1]["end"] = [f"r{i}"]
    return steps, where


def batch_trace(prompts, batches, tails):
    """Prompts (all but the last tails[i] tokens) in one step, then one token each; a request
    ends after its last token while the others go on."""
    steps, rows = [], {i: [] for i in range(len(prompts))}     # rows[i] = [(step, row)] per position
    for batch in batches:
        heads = {i: len(prompts[i]) - tails[i] for i in batch}
        ents, at = [], 0
        for i in batch:
            ents.append({"id": f"r{i}", "tokens": prompts[i][:heads[i]], "want": list(range(heads[i]))})
            rows[i] += [(len(steps), at + k) for k in range(heads[i])]
            at += heads[i]
        steps.append({"step": len(steps), "entries": ents, "end": [f"r{i}" for i in batch if tails[i] == 0]})
        k, live = 0, [i for i in batch if tails[i] > 0]
        while live:
            ents = [{"id": f"r{i}", "tokens": [prompts[i][heads[i] + k]], "want": [0]} for i in live]
            for r, i in enumerate(live):
                rows[i].append((len(steps), r))
            k += 1
            steps.append({"step": len(steps), "entries": ents, "end": [f"r{i}" for i in live if tails[i] == k]})
            live = [i for i in live if tails[i] > k]
    return steps, rows


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("A", "bfloat16"), ("B", "float32"), ("B", "bfloat16")])
def test_replay_three_ways(tmp_path, name, dtype):
    cfg = TINY[name]
    vocab = cfg["vocab_size"]
    folder = make_folder(tmp_path, cfg, seed=21, dtype=dtype)
    lengths = [5, 40, 97, 150] if name == "A" else [1, 33, 64, 140]
    prompts = prompts_for(cfg, lengths, seed=2)
    rnd = P.bf16_rounding if dtype == "bfloat16" else P.no_rounding
    w = plain_weights(folder)
    want = [P.forward(cfg, w, p, rnd) for p in prompts]

    out = str(tmp_path / "whole")
    replay(folder, dtype, whole_trace(prompts), out, max_tokens=192)          # one request at a time: 150 -> 192
    for i in range(len(prompts)):
        compare(read(out, i, vocab), want[i], dtype, f"whole, request {i}")

    out = str(tmp_path / "tail")
    steps, where = tail_trace(prompts)
    replay(folder, dtype, steps, out, max_tokens=192)
    for i in range(len(prompts)):
        got = torch.cat([read(out, s, vocab) for s in where[i]])
        compare(got, want[i], dtype, f"last 32 tokens one by one, request {i}")

    out = str(tmp_path / "batch")
    tails = {i: min(t, len(prompts[i]) - 1) for i, t in {0: 2, 1: 9, 2: 0, 3: 17}.items()}
    steps, rows = batch_trace(prompts, [[3, 0], [1, 2]], tails)
    # live at once: 150 + 5 -> 192 + 64; then 40 + 97 -> 64 + 128
    replay(folder, dtype, steps, out, max_tokens=256)
    files = {}
    for i in range(len(prompts)):
        got = []
        for s, r in rows[i]:
            if s not in files:
                files[s] = read(out, s, vocab)
            got.append(files[s][r])
        compare(torch.stack(got), want[i], dtype, f"unequal batches, request {i}")
    assert not os.path.exists(os.path.join(out, "nothing.f32"))


def test_step_without_wanted_rows_writes_no_file(tmp_path):
    cfg = TINY["A"]
    folder = make_folder(tmp_path, cfg, seed=21, dtype="float32")
    out = str(tmp_path / "o")
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": [1, 2, 3], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [4], "want": [0]}], "end": ["a"]}]
    replay(folder, "float32", steps, out, max_tokens=64)
    assert sorted(os.listdir(out)) == ["1.f32"]
    ref = P.forward(cfg, plain_weights(folder), [1, 2, 3, 4])
    compare(read(out, 1, cfg["vocab_size"]), ref[3:], "float32", "row after an unwanted prompt")
