"""The generation loop on workloads drawn at random: more requests than slots, prompts of unequal
lengths (some longer than a page), a cache so small that batches follow one another, stop tokens
that some requests hit at once and some never, with and without running ahead of the host.  Greedy
output equals the plain implementation's loop (the whole sequence run again for every token); with
a temperature, the two loops give the same tokens and a request's tokens do not depend on the
batch it ran in."""
import numpy as np
import pytest

from helpers import TINY, WEIGHT_STD
from plain import mistral_plain as P

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def models():
    import torch
    from inference_engine_rust_b200 import LoadedModel
    from inference_engine_rust_b200.weights import RandomSource
    out = {}
    for name in ("A", "B"):
        cfg = TINY[name]
        model = LoadedModel.random(cfg, seed=77, dtype="float32", std=WEIGHT_STD)
        src = RandomSource(model.model.expected_tensors(), 77, WEIGHT_STD, dtype=torch.float32)
        out[name] = (cfg, model, {n: src.get(n) for n in src.names()})
    return out


@pytest.mark.parametrize("name,seed", [("A", 0), ("B", 1), ("A", 2)])
def test_random_workload_greedy(models, name, seed):
    cfg, model, w = models[name]
    rng = np.random.default_rng(seed)
    n_req = int(rng.integers(5, 10))
    lengths = [int(rng.choice([1, 3, 9, 30, 62, 66, 90])) for _ in range(n_req)]
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in lengths]
    new = int(rng.integers(3, 9))
    free_run = [P.generate_greedy(cfg, w, p, new) for p in prompts]
    # stop tokens taken from what the requests would say: one at once, one in the middle, one that nobody says
    stop = {free_run[0][0], free_run[1][new // 2], cfg["vocab_size"] - 1}
    want = [P.generate_greedy(cfg, w, p, new, stop_ids=stop) for p in prompts]
    slots = int(rng.integers(2, 4))
    for run_ahead in (True, False):
        session = model.session(max_tokens=64 * 2 * slots, max_sequences=slots, poison_cache=True)
        res = session.generate(prompts, max_new_tokens=new, stop_ids=stop, full=True, run_ahead=run_ahead)
        assert [r.tokens for r in res] == want, f"run_ahead={run_ahead}"
        assert [r.finish_reason for r in res] == ["stop" if len(t) < new else "length" for t in want]
        session.engine.cache.check()
        assert session.engine.cache.slots.free_count == session.engine.cache.n_slots


@pytest.mark.parametrize("name,seed", [("A", 5), ("B", 6)])
def test_random_workload_with_a_temperature(models, name, seed):
    cfg, model, w = models[name]
    rng = np.random.default_rng(seed)
    lengths = [int(rng.choice([2, 8, 33, 64, 70])) for _ in range(6)]
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in lengths]
    ids = [int(i) for i in rng.permutation(100)[:6]]
    runs = []
    for slots, run_ahead, order in ((3, True, range(6)), (2, False, range(6)), (6, True, reversed(range(6)))):
        order = list(order)
        session = model.session(max_tokens=64 * 2 * slots, max_sequences=slots, poison_cache=True)
        out = session.generate([prompts[i] for i in order], max_new_tokens=7, temperature=0.9, seed=123, stop_ids=[],
                               request_ids=[ids[i] for i in order], run_ahead=run_ahead)
        by_request = [None] * 6
        for i, toks in zip(order, out):
            by_request[i] = toks
        runs.append(by_request)
    assert runs[0] == runs[1] == runs[2]
    assert len({tuple(t) for t in runs[0]}) > 1


@pytest.mark.parametrize("run_ahead", [True, False])
def test_the_context_limit_ends_a_request(models, run_ahead):
    """A cache whose sequences hold at most L positions: a request ends with the token chosen from the last
    position that fits ("context"), the others end by their own length; tokens equal the plain loop's."""
    cfg, model, w = models["A"]
    rng = np.random.default_rng(11)
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in (60, 10, 63)]
    limit, new = 66, 9
    session = model.session(max_tokens=64 * 2 * 3, max_sequences=3, max_seq_len=limit, poison_cache=True)
    res = session.generate(prompts, max_new_tokens=new, stop_ids=[], full=True, run_ahead=run_ahead)
    for p, r in zip(prompts, res):
        fits = min(new, limit - len(p) + 1)               # the token after the last position is still chosen
        assert r.tokens == P.generate_greedy(cfg, w, p, fits)
        assert r.finish_reason == ("length" if fits == new else "context")
    session.engine.cache.check()
    assert session.engine.cache.slots.free_count == session.engine.cache.n_slots
