"""Decisions of the generation loop, with a scripted engine in place of the device."""
import os

import pytest

from inference_engine_rust_b200.engine.generate import generate, plan_batches, run_batch, run_batch_ahead


class ScriptedEngine:
    """Stands where the engine stands.  'Logits' are the list of (slot, tokens so far)."""

    def __init__(self, n_slots):
        self.free = list(range(n_slots - 1, -1, -1))
        self.held = {}
        self.steps = []          # (kind, [(slot, n_tokens)])
        self.opened = []

    def open_sequence(self):
        s = self.free.pop()
        self.held[s] = []
        self.opened.append(s)
        return s

    def close_sequence(self, slot):
        assert slot in self.held, "closed twice"
        del self.held[slot]
        self.free.append(slot)

    def step(self, entries, want="last"):
        assert want == "last"
        lens = [len(t) for _, t in entries]
        first = all(len(self.held[s]) == 0 for s, _ in entries)
        assert first or all(n == 1 for n in lens), "mixed step"
        for s, t in entries:
            self.held[s].extend(t)
        self.steps.append(("prompt" if first and any(n > 1 for n in lens) else "decode", [(s, len(t)) for s, t in entries]))
        return [(s, list(self.held[s])) for s, _ in entries]


def scripted_sampler(script):
    """script[request] = tokens it will be given, in order."""
    calls = []

    def sampler(logits, request_ids, steps):
        calls.append((list(request_ids), list(steps)))
        return [script[r][st] for r, st in zip(request_ids, steps)]
    sampler.calls = calls
    return sampler


class AheadEngine(ScriptedEngine):
    """A scripted engine that also takes a step's tokens 'from the device': here a list that the
    scripted sampler made, of which the rows named are used."""

    def step_tokens_on_device(self, slots, tokens, rows=None, want="last"):
        rows = list(range(len(slots))) if rows is None else list(rows)
        assert len(rows) == len(slots) and rows == sorted(set(rows))
        return self.step([(s, [tokens[r]]) for s, r in zip(slots, rows)], want)


class AheadSampler:
    """The scripted sampler with the two calls of the run-ahead loop.  `wait()` hands the ids out
    and notes how many steps the engine had run by then."""

    def __init__(self, script, engine=None):
        self.script, self.engine, self.calls, self.waits = script, engine, [], []

    def __call__(self, logits, request_ids, steps):
        return self.sample_device(logits, request_ids, steps)

    def sample_device(self, logits, request_ids, steps):
        self.calls.append((list(request_ids), list(steps)))
        return [self.script[r][st] if st < len(self.script[r]) else 0 for r, st in zip(request_ids, steps)]

    def read_async(self, tokens):
        outer = self

        class Pending:
            def wait(self):
                outer.waits.append(len(outer.engine.steps) if outer.engine else None)
                return list(tokens)
        return Pending()


CASES = [
    # script, prompts, max_new_tokens, stop ids, max_seq_len
    ({0: [10, 11, 2, 99], 1: [2], 2: [20, 21, 22, 23, 24]}, [[1, 5], [1, 6, 7], [1]], 4, {2}, 100),
    ({0: [5, 6, 7]}, [[1, 2, 3]], 3, set(), 100),
    ({0: [5, 6, 7, 8, 9]}, [[1, 2, 3]], 10, set(), 5),
    ({0: [5], 1: [6]}, [[1], [1, 2]], 1, set(), 100),
    ({0: [7, 7, 2], 1: [2, 9], 2: [8, 2, 8], 3: [1, 1, 1, 1, 1, 2]}, [[1], [2, 2], [3, 3, 3], [4]], 6, {2}, 100),
    ({0: [3, 3, 3, 3], 1: [4, 2, 4, 4]}, [[1] * 6, [1] * 2], 9, {2}, 8),      # one ends by context, one on a stop
]


@pytest.mark.parametrize("script,prompts,max_new,stop,max_len", CASES)
def test_running_ahead_gives_the_plain_loop_s_results(script, prompts, max_new, stop, max_len):
    """Same tokens, reasons, token callbacks in the same order, every slot given back; the only
    extra work is one row-step for each sequence that ends on a stop token."""
    ids = list(range(len(prompts)))
    plain_eng, plain_seen = ScriptedEngine(len(prompts)), []
    plain = run_batch(plain_eng, scripted_sampler({r: t + [0] * 4 for r, t in script.items()}), prompts, ids,
                      max_new, stop, max_len, on_token=lambda r, t: plain_seen.append((r, t)))
    eng, seen = AheadEngine(len(prompts)), []
    sampler = AheadSampler(script, eng)
    ahead = run_batch_ahead(eng, sampler, prompts, ids, max_new, stop, max_len, on_token=lambda r, t: seen.append((r, t)))
    assert [(r.tokens, r.finish_reason) for r in ahead] == [(r.tokens, r.finish_reason) for r in plain]
    assert seen == plain_seen
    assert not eng.held and sorted(eng.free) == list(range(len(prompts)))
    rows_plain = sum(len(e) for _, e in plain_eng.steps[1:])
    rows_ahead = sum(len(e) for _, e in eng.steps[1:])
    stopped_after_start = sum(1 for r in plain if r.finish_reason == "stop")
    assert rows_plain <= rows_ahead <= rows_plain + stopped_after_start
    # the host reads the ids of step k only after step k + 1 was launched (except at the very end)
    for k, steps_run in enumerate(sampler.waits[:-1]):
        assert steps_run == k + 2, "the next step was not launched before the host waited"


def test_running_ahead_equals_the_plain_loop_on_random_scripts():
    """Three hundred random batches: sizes, prompt lengths, limits, stop tokens that fall anywhere
    (also on the first token, also for every sequence at once)."""
    import random
    rnd = random.Random(7)
    for case in range(300):
        n = rnd.randint(1, 6)
        max_new = rnd.randint(1, 9)
        prompts = [[1] * rnd.randint(1, 12) for _ in range(n)]
        max_len = rnd.choice([100, max(len(p) for p in prompts) + rnd.randint(0, 6)])
        stop = set(rnd.sample(range(2, 8), rnd.randint(0, 3)))
        script = {r: [rnd.randint(2, 12) for _ in range(max_new + 1)] for r in range(n)}
        ids = list(range(n))
        e1, seen1 = ScriptedEngine(n), []
        plain = run_batch(e1, scripted_sampler(script), prompts, ids, max_new, stop, max_len,
                          on_token=lambda r, t: seen1.append((r, t)))
        e2, seen2 = AheadEngine(n), []
        ahead = run_batch_ahead(e2, AheadSampler(script, e2), prompts, ids, max_new, stop, max_len,
                                on_token=lambda r, t: seen2.append((r, t)))
        assert [(r.tokens, r.finish_reason) for r in ahead] == [(r.tokens, r.finish_reason) for r in plain], case
        assert seen1 == seen2 and not e2.held and len(e2.free) == n, case
        # what each slot was fed is what the plain loop fed it, plus at most one token after a stop
        for (k1, s1), (k2, s2) in zip(e1.steps, e2.steps):
            assert k1 == k2 and set(s1) <= set(s2), case


def test_running_ahead_is_chosen_by_generate_when_both_sides_can():
    eng = AheadEngine(2)
    sampler = AheadSampler({i: [30 + i, 40 + i, 2] for i in range(5)}, eng)
    res = generate(eng, sampler, [[1, i] for i in range(5)], 8, stop_ids=[2], max_tokens=64 * 2,
                   max_sequences=2, max_seq_len=64, page_tokens=64)
    assert [r.tokens for r in res] == [[30 + i, 40 + i] for i in range(5)] and sampler.waits
    eng2 = AheadEngine(2)
    sampler2 = AheadSampler({i: [30 + i, 40 + i, 2] for i in range(5)}, eng2)
    res2 = generate(eng2, sampler2, [[1, i] for i in range(5)], 8, stop_ids=[2], max_tokens=64 * 2,
                    max_sequences=2, max_seq_len=64, page_tokens=64, run_ahead=False)
    assert [r.tokens for r in res2] == [r.tokens for r in res] and not sampler2.waits


def test_stop_token_is_not_kept_and_shorter_sequences_end_earlier():
    eng = ScriptedEngine(4)
    script = {0: [10, 11, 2, 99], 1: [2], 2: [20, 21, 22, 23, 24]}
    res = run_batch(eng, scripted_sampler(script), [[1, 5], [1, 6, 7], [1]], [0, 1, 2], 4, {2}, 100)
    assert [r.tokens for r in res] == [[10, 11], [], [20, 21, 22, 23]]
    assert [r.finish_reason for r in res] == ["stop", "stop", "length"]
    assert eng.steps[0] == ("prompt", [(0, 2), (1, 3), (2, 1)])
    assert [len(e) for _, e in eng.steps[1:]] == [2, 2, 1]           # batch shrinks; no step after the last token
    assert not eng.held and sorted(eng.free) == [0, 1, 2, 3]


def test_no_forward_after_the_last_kept_token():
    eng = ScriptedEngine(1)
    res = run_batch(eng, scripted_sampler({0: [5, 6, 7]}), [[1, 2, 3]], [0], 3, set(), 100)
    assert res[0].tokens == [5, 6, 7] and len(eng.steps) == 3        # prompt + 2 decode steps


def test_context_limit_ends_a_sequence():
    eng = ScriptedEngine(1)
    res = run_batch(eng, scripted_sampler({0: [5, 6, 7, 8, 9]}), [[1, 2, 3]], [0], 10, set(), 5)
    assert res[0].finish_reason == "context" and res[0].tokens == [5, 6, 7]   # 3 + 2 positions run, third token has no room


def test_zero_new_tokens_runs_nothing():
    eng = ScriptedEngine(1)
    res = run_batch(eng, scripted_sampler({}), [[1]], [0], 0, set(), 10)
    assert res[0].tokens == [] and not eng.steps and not eng.opened


def test_slots_come_back_when_a_step_fails():
    class Failing(ScriptedEngine):
        def step(self, entries, want="last"):
            if self.steps:
                raise RuntimeError("boom")
            return super().step(entries, want)
    eng = Failing(3)
    with pytest.raises(RuntimeError):
        run_batch(eng, scripted_sampler({0: [5, 5], 1: [6, 6]}), [[1], [1]], [0, 1], 5, set(), 100)
    assert not eng.held and len(eng.free) == 3


def test_plan_batches():
    kw = dict(max_tokens=64 * 6, max_sequences=3, max_seq_len=256, page_tokens=64)
    assert plan_batches([10, 10, 10, 10], 20, **kw) == [[0, 1, 2], [3]]              # slot bound
    assert plan_batches([100, 100, 10], 60, **kw) == [[0, 1], [2]]                    # 192 + 192 = 384 tokens
    assert plan_batches([10, 10, 10], 5, max_batch=2, **kw) == [[0, 1], [2]]
    assert plan_batches([250], 100, **kw) == [[0]]                                    # capped by max_seq_len
    for bad in ([0], [257]):
        with pytest.raises(ValueError):
            plan_batches(bad, 5, **kw)
    with pytest.raises(ValueError):
        plan_batches([200], 100, max_tokens=128, max_sequences=3, max_seq_len=256, page_tokens=64)


def test_batches_one_after_another_reuse_slots_and_keep_order():
    eng = ScriptedEngine(2)
    script = {i: [30 + i, 40 + i, 2] for i in range(5)}
    sampler = scripted_sampler(script)
    res = generate(eng, sampler, [[1, i] for i in range(5)], 8, stop_ids=[2], max_tokens=64 * 2,
                   max_sequences=2, max_seq_len=64, page_tokens=64)
    assert [r.tokens for r in res] == [[30 + i, 40 + i] for i in range(5)]
    assert [r.request for r in res] == list(range(5))
    assert eng.opened == [0, 1, 1, 0, 0] or len(set(eng.opened)) == 2                 # two slots serve five requests
    assert sampler.calls[0] == ([0, 1], [0, 0]) and sampler.calls[3] == ([2, 3], [0, 0])
    assert not eng.held


def test_request_ids_reach_the_sampler():
    eng = ScriptedEngine(2)
    sampler = scripted_sampler({7: [5], 9: [6]})
    generate(eng, sampler, [[1], [1]], 1, max_tokens=128, max_sequences=2, max_seq_len=64, page_tokens=64,
             request_ids=[7, 9])
    assert sampler.calls == [([7, 9], [0, 0])]


def test_bench_summaries_and_arguments(capsys):
    """The bench suite's statistics (src/bin/bench_compare.rs:234-300) and its argument checks."""
    from inference_engine_rust_b200 import bench_metrics as M
    from inference_engine_rust_b200.cli import main
    assert M.median([3.0, 1.0, 2.0]) == 2.0 and M.median([4.0, 1.0, 2.0, 3.0]) == 2.5 and M.median([]) == 0.0
    vals = [float(v) for v in range(1, 21)]
    assert M.percentile(vals, 0.95) == 19.0 and M.percentile(vals, 0.0) == 1.0 and M.percentile(vals, 1.0) == 20.0
    runs = [{"decode_tokens_per_sec": t, "decode_elapsed_ms": 1000.0 / t, "decode_tokens": 8} for t in (10.0, 30.0, 20.0)]
    s = M.summarize_decode(runs)
    assert s["runs"] == 3 and s["decode_tokens_per_sec"] == {"median": 20.0, "p95": 30.0, "min": 10.0, "max": 30.0}
    with pytest.raises(ValueError):
        M.summarize_decode([])
    M.check_decode(runs[0], 10.0)
    with pytest.raises(RuntimeError, match="min-decode-tps"):
        M.check_decode(runs[0], 10.5)
    with pytest.raises(RuntimeError, match="zero"):
        M.check_decode(dict(runs[0], decode_tokens=0), None)
    assert main(["bench", "--runs", "4", "cold-start"]) == 2 and "at least 5" in capsys.readouterr().err
    assert main(["bench", "-p", "x y", "cold-start"]) == 2 and "token ids" in capsys.readouterr().err
    assert main(["bench", "-m", "/nonexistent/folder", "cold-start"]) == 1


def test_no_device_and_no_compiler_fail_loudly(monkeypatch, tmp_path):
    """Without a GPU the engine refuses to be built (there is no CPU path); without nvcc the
    kernels cannot be compiled and the build says where it looked."""
    import torch
    from inference_engine_rust_b200 import LoadedModel
    from inference_engine_rust_b200.csrc import build
    from inference_engine_rust_b200.csrc.bindings import KernelError
    if not torch.cuda.is_available():
        cfg = {"architectures": ["MistralForCausalLM"], "num_hidden_layers": 1, "hidden_size": 32,
               "num_attention_heads": 2, "num_key_value_heads": 1, "intermediate_size": 48, "vocab_size": 50,
               "rms_norm_eps": 1e-5, "max_position_embeddings": 64}
        model = LoadedModel.random(cfg, seed=0, dtype="float32", device="cpu")
        with pytest.raises(KernelError, match="no CUDA device"):
            model.session(max_tokens=64)
    monkeypatch.setenv("IERT_NVCC", str(tmp_path / "missing-nvcc"))
    monkeypatch.setenv("PATH", str(tmp_path))
    real = os.path.isfile
    monkeypatch.setattr(build.os.path, "isfile", lambda p: False if str(p).endswith("nvcc") else real(p))
    with pytest.raises(build.BuildError, match="nvcc not found"):
        build.find_nvcc()


@pytest.mark.parametrize("run", [run_batch, run_batch_ahead])
def test_slots_opened_before_a_failed_open_are_given_back(run):
    """Fewer free slots than prompts: the open that fails must not leak the slots opened before it."""
    class Full(Exception):
        pass

    class TwoSlots(AheadEngine):
        def open_sequence(self):
            if not self.free:
                raise Full("no slot is free")
            return super().open_sequence()

    eng = TwoSlots(2)
    sampler = AheadSampler({0: [5], 1: [6], 2: [7]}, eng)
    with pytest.raises(Full):
        run(eng, sampler, [[1], [2], [3]], [0, 1, 2], 4, set(), 100)
    assert eng.held == {} and sorted(eng.free) == [0, 1] and eng.steps == []
