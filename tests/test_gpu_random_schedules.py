"""One engine driven through a schedule drawn at random: prompt steps that open one to three new
sequences of unequal lengths (with all, the last, chosen or no logits wanted), one-token steps over
an arbitrary subset of the live sequences in an arbitrary order (the others stay where they are),
sequences closed at any time and their slots and pages taken again.  Every logit that comes back is
compared with the plain implementation's for that sequence and position: the logits at a position
depend neither on how the tokens were cut into steps, nor on what else was in the batch, nor on
where in the cache they lie."""
import os

import numpy as np
import pytest
import torch

from helpers import TINY, WEIGHT_STD, compare
from plain import mistral_plain as P

pytestmark = pytest.mark.gpu


# (a longer hunt: IERT_TEST_RANDOM_SCHEDULES=40 adds that many seeds for every tiny configuration)
CASES = [("A", 0), ("A", 1), ("B", 2), ("C", 3)] + [
    (name, 100 + i) for i in range(int(os.environ.get("IERT_TEST_RANDOM_SCHEDULES", "0"))) for name in "ABCD"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,seed", CASES)
def test_a_random_schedule_of_steps(name, seed, dtype):
    from inference_engine_rust_b200 import LoadedModel
    from inference_engine_rust_b200.weights import RandomSource
    cfg = TINY[name]
    model = LoadedModel.random(cfg, seed=31 + seed, dtype=dtype, std=WEIGHT_STD)
    src = RandomSource(model.model.expected_tensors(), 31 + seed, WEIGHT_STD, dtype=torch.float32)
    w = {n: src.get(n) for n in src.names()}
    if dtype == "bfloat16":
        w = {n: t.to(torch.bfloat16).float() for n, t in w.items()}
    if cfg.get("tie_word_embeddings"):
        w["lm_head.weight"] = w["model.embed_tokens.weight"]
    rnd = P.bf16_rounding if dtype == "bfloat16" else P.no_rounding
    rng = np.random.default_rng(seed)
    max_live, max_len = 4, 200
    eng = model.session(max_tokens=max_live * 256, max_sequences=max_live, max_seq_len=256, poison_cache=True).engine

    live = {}            # slot -> dict(tokens, fed, ref)
    checked = steps = 0

    def new_request():
        n = int(rng.choice([1, 2, 7, 31, 63, 64, 65, 100, 129, max_len]))
        tokens = rng.integers(0, cfg["vocab_size"], n).tolist()
        return dict(tokens=tokens, fed=0, ref=P.forward(cfg, w, tokens, rnd), rows=[], got=[])

    all_got, all_ref = [], []

    def retire(r):
        """A request leaves: the logits it got and the plain ones at the same positions join the pile that
        is compared when the schedule has ended (as one tensor: the bfloat16 bound on the mean error is
        a statement about many rows, not about one)."""
        if r["rows"]:
            all_got.append(torch.cat(r["got"]).float().cpu())
            all_ref.append(r["ref"][r["rows"]])

    while steps < 45:
        room = max_live - len(live)
        decodable = [s for s, r in live.items() if r["fed"] < len(r["tokens"])]
        action = rng.choice(["prompt", "decode", "decode", "close"])
        if action == "prompt" and room > 0:
            k = int(rng.integers(1, min(room, 3) + 1))
            entries, reqs, want_places = [], [], []
            for _ in range(k):
                r = new_request()
                slot = eng.open_sequence()
                # the prompt is a prefix of the request; the rest comes token by token
                cut = int(rng.integers(1, len(r["tokens"]) + 1))
                entries.append((slot, r["tokens"][:cut]))
                reqs.append((slot, r, cut))
            mode = rng.choice(["all", "last", "places", "none"])
            if mode == "places":
                want = [sorted(set(rng.integers(0, cut, size=min(cut, 3)).tolist())) for _, _, cut in reqs]
            else:
                want = None if mode == "none" else str(mode)
            out = eng.step(entries, want=want)
            at = 0
            for (slot, r, cut), places in zip(reqs, want if mode == "places" else [None] * k):
                rows = list(range(cut)) if mode == "all" else [cut - 1] if mode == "last" else places if mode == "places" else []
                if rows:
                    r["rows"] += rows
                    r["got"].append(out[at:at + len(rows)].clone())
                    at += len(rows)
                    checked += len(rows)
                r["fed"] = cut
                live[slot] = r
            assert out is None or at == out.shape[0]
        elif action == "decode" and decodable:
            k = int(rng.integers(1, len(decodable) + 1))
            chosen = [int(s) for s in rng.permutation(decodable)[:k]]
            out = eng.step([(s, [live[s]["tokens"][live[s]["fed"]]]) for s in chosen], want="last")
            for j, s in enumerate(chosen):
                r = live[s]
                r["rows"].append(r["fed"])
                r["got"].append(out[j:j + 1].clone())
                r["fed"] += 1
                checked += 1
        elif action == "close" and live:
            s = int(rng.choice(list(live)))
            eng.close_sequence(s)
            retire(live.pop(s))
        else:
            continue
        steps += 1
    eng.check_device()
    for s in list(live):
        retire(live.pop(s))
    eng.cache.check()
    assert checked > 40
    compare(torch.cat(all_got), torch.cat(all_ref), dtype, f"{checked} logits gathered over the schedule")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_two_sessions_of_one_model_do_not_disturb_each_other(dtype):
    """Two sessions of the same loaded model (shared weights, a cache and captured steps each), used in
    turns, and a third one made and dropped in between: every logit as the plain implementation has it."""
    import gc
    from inference_engine_rust_b200 import LoadedModel
    from inference_engine_rust_b200.weights import RandomSource
    cfg = TINY["B"]
    model = LoadedModel.random(cfg, seed=5, dtype=dtype, std=WEIGHT_STD)
    src = RandomSource(model.model.expected_tensors(), 5, WEIGHT_STD, dtype=torch.float32)
    w = {n: src.get(n) for n in src.names()}
    if dtype == "bfloat16":
        w = {n: t.to(torch.bfloat16).float() for n, t in w.items()}
    rnd = P.bf16_rounding if dtype == "bfloat16" else P.no_rounding
    rng = np.random.default_rng(9)
    seqs = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in (50, 71, 20, 66)]
    refs = [P.forward(cfg, w, s, rnd) for s in seqs]
    engines = [model.session(max_tokens=64 * 4, poison_cache=True).engine for _ in range(2)]
    owner = [0, 1, 0, 1]                                   # which engine runs which sequence
    slots, fed, got = [], [], [[] for _ in seqs]
    for i, s in enumerate(seqs):
        eng = engines[owner[i]]
        slot = eng.open_sequence()
        slots.append(slot)
        got[i].append(eng.step([(slot, s[:10])], want="all").clone())
        fed.append(10)
    for round_ in range(10):
        for e, eng in enumerate(engines):
            mine = [i for i in range(len(seqs)) if owner[i] == e]
            out = eng.step([(slots[i], [seqs[i][fed[i]]]) for i in mine], want="last")
            for r, i in enumerate(mine):
                got[i].append(out[r:r + 1].clone())
                fed[i] += 1
        if round_ == 3:                                    # a third session comes, steps (graphs and all) and goes
            other = model.session(max_tokens=64 * 2).engine
            s3 = other.open_sequence()
            other.step([(s3, seqs[0][:5])], want="last")
            for t in seqs[0][5:9]:
                other.step([(s3, [t])], want="last")
            del other
            gc.collect()
    for eng in engines:
        eng.check_device()
    for i in range(len(seqs)):
        compare(torch.cat(got[i]), refs[i][:fed[i]], dtype, f"sequence {i} in session {owner[i]}")
