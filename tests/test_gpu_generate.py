"""Generation through the Python entry point and the command line: greedy tokens equal the
plain implementation's (whole sequence run again for every token), stop tokens, batches one
after another, temperature sampling that does not depend on the batch."""
import json
import os
import subprocess
import sys

import pytest
import torch

from helpers import TINY, make_folder, plain_weights, prompts_for
from plain import mistral_plain as P

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def loaded(tmp_path_factory):
    from inference_engine_rust_b200 import LoadedModel
    out = {}
    root = tmp_path_factory.mktemp("gen")
    for name in ("A", "B"):
        folder = make_folder(root, TINY[name], seed=31, dtype="float32")
        out[name] = (folder, LoadedModel.load(folder, dtype="float32"), plain_weights(folder))
    return out


@pytest.mark.parametrize("name,lengths,new", [("A", [5, 11, 23], 8), ("B", [1, 7, 19, 40], 12)])
def test_greedy_equals_teacher_forcing(loaded, name, lengths, new):
    folder, model, w = loaded[name]
    cfg = TINY[name]
    prompts = prompts_for(cfg, lengths, seed=3)
    session = model.session(max_tokens=64 * 8, poison_cache=True)
    got = session.generate(prompts, max_new_tokens=new, stop_ids=[])
    want = [P.generate_greedy(cfg, w, p, new) for p in prompts]
    assert got == want
    session.engine.cache.check()
    assert session.engine.cache.slots.free_count == session.engine.cache.n_slots


def test_stop_tokens_and_batches_one_after_another(loaded):
    folder, model, w = loaded["A"]
    cfg = TINY["A"]
    prompts = prompts_for(cfg, [9, 4, 30, 17, 2, 12, 6], seed=4)
    free_run = [P.generate_greedy(cfg, w, p, 10) for p in prompts]
    stop = {free_run[0][3], free_run[2][0], free_run[5][7]}
    want = [P.generate_greedy(cfg, w, p, 10, stop_ids=stop) for p in prompts]
    session = model.session(max_tokens=64 * 3, max_sequences=3, poison_cache=True)   # three slots for seven requests
    res = session.generate(prompts, max_new_tokens=10, stop_ids=stop, full=True)
    assert [r.tokens for r in res] == want
    assert res[2].tokens == [] and res[2].finish_reason == "stop"
    assert [r.finish_reason for r in res] == ["stop" if len(t) < 10 else "length" for t in want]
    assert session.engine.steps_run > 3 * 1
    session.engine.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_running_ahead_changes_no_token(loaded, tmp_path, dtype):
    """The loop that feeds chosen ids from device memory and reads them one step behind against
    the loop that waits for them every step: greedy and temperature, stop tokens that end
    sequences in the middle of a batch, more requests than slots."""
    from inference_engine_rust_b200 import LoadedModel
    folder, model, w = loaded["A"]
    cfg = TINY["A"]
    if dtype == "bfloat16":
        model = LoadedModel.load(make_folder(tmp_path, cfg, seed=31, dtype="bfloat16"), dtype="bfloat16")
    prompts = prompts_for(cfg, [9, 4, 30, 17, 2, 12, 6, 70], seed=4)
    session = model.session(max_tokens=64 * 4, max_sequences=3, poison_cache=True)
    for temperature in (0.0, 0.9):
        free_run = session.generate(prompts, max_new_tokens=12, temperature=temperature, seed=5, stop_ids=[],
                                    run_ahead=False)
        stop = {free_run[0][3], free_run[2][0], free_run[5][7], free_run[7][11]}
        seen_a, seen_b = [], []
        plain = session.generate(prompts, max_new_tokens=12, temperature=temperature, seed=5, stop_ids=stop,
                                 full=True, run_ahead=False, on_token=lambda r, t: seen_a.append((r, t)))
        ahead = session.generate(prompts, max_new_tokens=12, temperature=temperature, seed=5, stop_ids=stop,
                                 full=True, on_token=lambda r, t: seen_b.append((r, t)))
        assert [(r.tokens, r.finish_reason) for r in ahead] == [(r.tokens, r.finish_reason) for r in plain]
        assert seen_a == seen_b and any(r.finish_reason == "stop" for r in plain)
        session.engine.cache.check()
        assert session.engine.cache.slots.held_count == 0


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_generation_across_a_page_boundary_and_a_ring_wrap(loaded, tmp_path, name, dtype):
    """Prompts of 60 and 125 tokens and 12 new tokens: decoding crosses positions 64 and 128, so a
    page is taken in the middle of a run (with the device one step ahead of the host, the page
    table is brought up to date while the step before still runs) and, with Tiny A's window of
    16, the 64-position ring wraps.  A third, short request ends early.  Both loops, poisoned
    cache.  Greedy: the plain implementation's tokens (float32; in bfloat16 the two loops agree
    and every token is the argmax of the plain logits within the tolerance).  Temperature: the
    two loops agree."""
    from inference_engine_rust_b200 import LoadedModel
    folder, model, w = loaded[name]
    cfg = TINY[name]
    if dtype == "bfloat16":
        folder = make_folder(tmp_path, cfg, seed=31, dtype="bfloat16")
        model = LoadedModel.load(folder, dtype="bfloat16")
        w = plain_weights(folder)
    prompts = prompts_for(cfg, [60, 125, 3], seed=13)
    session = model.session(max_tokens=64 * 6, max_sequences=3, poison_cache=True)
    by_loop = {}
    for run_ahead in (False, True):
        res = session.generate(prompts, max_new_tokens=12, stop_ids=[], full=True, run_ahead=run_ahead)
        by_loop[run_ahead] = [r.tokens for r in res]
        assert all(len(r.tokens) == 12 and r.finish_reason == "length" for r in res)
        session.engine.cache.check()
        assert session.engine.cache.slots.held_count == 0
    assert by_loop[True] == by_loop[False]
    if dtype == "float32":
        assert by_loop[True] == [P.generate_greedy(cfg, w, p, 12) for p in prompts]
    else:
        for p, toks in zip(prompts, by_loop[True]):
            logits = P.forward(cfg, w, list(p) + toks[:-1], P.bf16_rounding)[len(p) - 1:]
            for row, tok in zip(logits, toks):       # the chosen token is the best, or within rounding of the best
                assert row[tok] >= row.max() - 2.0 ** -6 * 2 * row.abs().max()
    # a stop token met in the middle of the second page, and sampling: the loops still agree
    stop = {by_loop[True][0][7], by_loop[True][1][5]}
    for temperature in (0.0, 0.8):
        a = session.generate(prompts, max_new_tokens=12, temperature=temperature, seed=3, stop_ids=stop, full=True,
                             run_ahead=False)
        b = session.generate(prompts, max_new_tokens=12, temperature=temperature, seed=3, stop_ids=stop, full=True)
        assert [(r.tokens, r.finish_reason) for r in a] == [(r.tokens, r.finish_reason) for r in b]
    assert session.engine.cache.slots.held_count == 0


def test_a_step_takes_its_tokens_from_device_memory(loaded):
    """`step_tokens_on_device` against `step` with the same ids from the host: the same logits to
    the bit, also when the rows used are not all of the tensor and when graphs are off; what it
    cannot run is refused on the host."""
    from inference_engine_rust_b200 import StepError
    folder, model, w = loaded["B"]
    cfg = TINY["B"]
    prompts = prompts_for(cfg, [4, 9, 17], seed=6)
    ids = torch.tensor([5, 77, 300, 9, 41], dtype=torch.int32, device="cuda:0")
    for use_graphs in (True, False):
        a = model.session(max_tokens=512, use_graphs=use_graphs)
        b = model.session(max_tokens=512, use_graphs=use_graphs)
        a.prefill(prompts)
        b.prefill(prompts)
        for rows in ([0, 1, 2], [1, 2, 4], [4, 1, 3]):
            want = a.decode_tokens([int(ids[r]) for r in rows])
            got = b.engine.step_tokens_on_device(b._slots, ids, rows)
            assert torch.equal(got, want)
        assert torch.equal(b.decode_tokens_on_device(ids[:3]), a.decode_tokens([5, 77, 300]))
        b.engine.check_device()
        with pytest.raises(StepError):
            b.engine.step_tokens_on_device(b._slots, ids.long())
        with pytest.raises(StepError):
            b.engine.step_tokens_on_device(b._slots, ids, [0, 1, 5])
        with pytest.raises(StepError):
            b.engine.step_tokens_on_device(b._slots[:2], ids, [0, 1, 2])
        # an id outside the vocabulary is reported by the device
        bad = torch.tensor([1, cfg["vocab_size"], 2], dtype=torch.int32, device="cuda:0")
        b.decode_tokens_on_device(bad)
        from inference_engine_rust_b200.engine.engine import DeviceFault
        with pytest.raises(DeviceFault):
            b.engine.check_device()
        a.reset()
        b.reset()


def test_default_stop_is_the_configured_eos(loaded):
    folder, model, w = loaded["B"]
    cfg = TINY["B"]
    p = prompts_for(cfg, [6], seed=8)[0]
    free_run = P.generate_greedy(cfg, w, p, 6)
    from inference_engine_rust_b200 import LoadedModel
    cfg2 = dict(cfg, eos_token_id=free_run[2])
    folder2 = os.path.join(os.path.dirname(folder), "eos_variant")
    os.makedirs(folder2, exist_ok=True)
    with open(os.path.join(folder2, "config.json"), "w") as f:
        json.dump(cfg2, f)
    if not os.path.exists(os.path.join(folder2, "model.safetensors")):
        os.link(os.path.join(folder, "model.safetensors"), os.path.join(folder2, "model.safetensors"))
    m2 = LoadedModel.load(folder2, dtype="float32")
    assert m2.session(max_tokens=128).generate([p], max_new_tokens=6) == [free_run[:free_run.index(free_run[2])]]


def test_temperature_sampling_is_per_request(loaded):
    folder, model, w = loaded["A"]
    cfg = TINY["A"]
    prompts = prompts_for(cfg, [7, 3, 15], seed=5)
    session = model.session(max_tokens=64 * 6)
    together = session.generate(prompts, max_new_tokens=6, temperature=0.8, seed=99, stop_ids=[])
    alone = [session.generate([p], max_new_tokens=6, temperature=0.8, seed=99, stop_ids=[], request_ids=[i])[0]
             for i, p in enumerate(prompts)]
    assert together == alone
    other = session.generate(prompts, max_new_tokens=6, temperature=0.8, seed=100, stop_ids=[])
    assert other != together
    # each token follows the plain inverse-CDF rule for that request's draw
    for i, (p, toks) in enumerate(zip(prompts, together)):
        ids = list(p)
        for step, tok in enumerate(toks):
            logits = P.forward(cfg, w, ids)[-1]
            cdf = P.temperature_cdf(logits, 0.8)
            u = P.uniform_draw(99, i, step)
            lo = float(cdf[tok - 1]) if tok > 0 else 0.0
            assert lo - 1e-4 <= u <= float(cdf[tok]) + 1e-4
            ids.append(tok)


def test_session_calls_in_the_reference_manner(loaded):
    folder, model, w = loaded["B"]
    cfg = TINY["B"]
    prompts = prompts_for(cfg, [4, 9], seed=6)
    s = model.session(max_tokens=256)
    logits = s.prefill(prompts)
    host = s.logits_last_token(logits)
    assert len(host) == 2 and len(host[0]) == cfg["vocab_size"]
    nxt = [P.sample_greedy(r) for r in host]
    assert nxt == [P.sample_greedy(P.forward(cfg, w, p)[-1].tolist()) for p in prompts]
    logits = s.decode_tokens([nxt[0], None])          # the second sequence ends
    ref = P.forward(cfg, w, prompts[0] + [nxt[0]])[-1]
    assert torch.allclose(logits[0].cpu(), ref, atol=2e-4, rtol=2e-4)
    with pytest.raises(RuntimeError):
        s.prefill(prompts)
    s.reset()
    assert s.engine.cache.slots.held_count == 0
    from inference_engine_rust_b200 import StepError
    for bad in ([[]], [[cfg["vocab_size"]]], [[-1]]):
        with pytest.raises(StepError):
            s.prefill(bad)
        assert s.engine.cache.slots.held_count == 0


def test_command_line(loaded):
    folder, model, w = loaded["A"]
    cfg = TINY["A"]
    p = prompts_for(cfg, [6], seed=7)[0]
    want = P.generate_greedy(cfg, w, p, 5)
    cmd = [sys.executable, "-m", "inference_engine_rust_b200", "-m", folder, "--dtype", "float32", "-n", "5",
           "--stop-token", "-1", " ".join(map(str, p))]
    out = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    assert out.stdout.strip().split() == [str(t) for t in want]
    out = subprocess.run(cmd[:-1], cwd=ROOT, input=",".join(map(str, p)) + "\n", capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and out.stdout.strip().split() == [str(t) for t in want]
    bad = subprocess.run(cmd[:-1] + [""], cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert bad.returncode != 0 and "prompt" in bad.stderr.lower()


def test_command_line_runs_a_file_of_unequal_requests(loaded, tmp_path):
    """`--prompt-file`: one request per line becomes one generation call, whose batches hold
    requests of unequal lengths; one output line per request, in order.  With `--max-batch 2` the
    three requests run as two batches one after the other (slots used again)."""
    folder, model, w = loaded["B"]
    cfg = TINY["B"]
    prompts = prompts_for(cfg, [7, 1, 19], seed=11)
    want = [P.generate_greedy(cfg, w, p, 6) for p in prompts]
    f = tmp_path / "requests.txt"
    f.write_text("# three requests\n" + "\n".join(",".join(map(str, p)) for p in prompts) + "\n\n")
    base = [sys.executable, "-m", "inference_engine_rust_b200", "-m", folder, "--dtype", "float32", "-n", "6",
            "--stop-token", "-1"]
    for extra in ([], ["--max-batch", "2"]):
        out = subprocess.run(base + extra + ["--prompt-file", str(f)], cwd=ROOT, capture_output=True, text=True, timeout=300)
        assert out.returncode == 0, out.stderr
        lines = out.stdout.strip().splitlines()
        assert [ln.split() for ln in lines] == [[str(t) for t in r] for r in want]
    # --max-context ends a request when its sequence is full: of 22 positions the prompt takes 19, three
    # new tokens are run, and the fourth is still chosen (from the last position's logits) and kept
    out = subprocess.run(base + ["--max-context", "22", "--prompt-file", str(f)], cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    lines = [ln.split() for ln in out.stdout.strip().splitlines()]
    assert lines[0] == [str(t) for t in want[0]] and lines[2] == [str(t) for t in want[2][:4]]
    both = subprocess.run(base + ["--prompt-file", str(f), "1 2"], cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert both.returncode == 2 and "either" in both.stderr


def test_command_line_random_preset_and_lenient_loading(loaded, tmp_path):
    """`--random PRESET --seed N` needs no folder and gives the tokens of the same seeded weights
    written to a folder; a folder with a tensor the model does not use is refused unless
    `--ignore-extra-tensors` is given; a folder without the output head runs with the tied one."""
    from safetensors.torch import load_file, save_file
    from inference_engine_rust_b200 import write_random_model
    from inference_engine_rust_b200.config import preset
    cfg = preset("tiny-a")
    d = str(tmp_path / "tiny_a")
    write_random_model(d, cfg, seed=9, dtype="bfloat16", std=0.02)
    prompt = "5 9 200 31"
    tail = ["--dtype", "float32", "-n", "5", "--stop-token", "-1", prompt]
    run = lambda args: subprocess.run([sys.executable, "-m", "inference_engine_rust_b200"] + args, cwd=ROOT,
                                      capture_output=True, text=True, timeout=300)
    a = run(["--random", "tiny-a", "--seed", "9"] + tail)
    assert a.returncode == 0, a.stderr
    assert len(a.stdout.split()) == 5
    assert run(["--random", "tiny-a", "--seed", "9"] + tail).stdout == a.stdout, "same seed, same tokens"
    assert run(["--random", "tiny-c"] + tail).returncode == 2               # no such preset
    assert run(["--random", "tiny-a", "-m", d] + tail).returncode == 2      # one or the other
    # extras
    t = {k: v.clone() for k, v in load_file(os.path.join(d, "model.safetensors")).items()}   # not the file's mapping
    want = P.generate_greedy(cfg, {k: v.float() for k, v in t.items()}, [5, 9, 200, 31], 5)
    t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    save_file(t, os.path.join(d, "model.safetensors"))
    strict = run(["-m", d] + tail)
    assert strict.returncode == 1 and "unexpected (1)" in strict.stderr and "rotary_emb" in strict.stderr
    lenient = run(["-m", d, "--ignore-extra-tensors"] + tail)
    assert lenient.returncode == 0, lenient.stderr
    assert lenient.stdout.split() == [str(x) for x in want] and "ignored" in lenient.stderr
    # no output head in the folder: tied to the embedding
    del t["lm_head.weight"], t["model.layers.0.self_attn.rotary_emb.inv_freq"]
    save_file(t, os.path.join(d, "model.safetensors"))
    tied = run(["-m", d] + tail)
    assert tied.returncode == 0, tied.stderr
    w_tied = {k: v.float() for k, v in t.items()}
    w_tied["lm_head.weight"] = w_tied["model.embed_tokens.weight"]
    assert tied.stdout.split() == [str(x) for x in P.generate_greedy(cfg, w_tied, [5, 9, 200, 31], 5)]
    assert "tied" in tied.stderr


def test_bench_subcommand(loaded, capsys):
    """The reference's bench suite (cold start, interactive TTFT, decode throughput) through the
    command line's own entry, on a tiny model; the decode loop it times is the greedy loop."""
    from inference_engine_rust_b200 import bench_metrics as M
    from inference_engine_rust_b200.cli import main
    folder, model, w = loaded["A"]
    rc = main(["bench", "-m", folder, "--dtype", "float32", "--json", "-p", "3 9 27 81", "all", "--decode-tokens", "6"])
    assert rc == 0
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert out["suite"] == "all" and len(out["runs"]["decode"]) == 5
    d = out["runs"]["decode"][0]
    assert d["prompt_token_count"] == 4 and d["decode_tokens"] == 6 and d["decode_tokens_per_sec"] > 0
    assert out["summary"]["decode"]["decode_tokens_per_sec"]["min"] <= out["summary"]["decode"]["decode_tokens_per_sec"]["median"]
    c = out["runs"]["cold"][0]
    assert c["cold_ttft_ms"] >= c["tensor_load_ms"] + c["prompt_eval_ms"]
    i = out["runs"]["interactive"][0]
    assert abs(i["ttft_infer_ms"] - i["prompt_eval_ms"] - i["lm_head_sample_ms"]) < 1e-6
    # a floor no run can meet fails the command, as in the reference
    rc = main(["bench", "-m", folder, "--dtype", "float32", "--min-decode-tps", "1e12", "-p", "3 9 27",
               "decode-throughput", "-n", "3"])
    assert rc == 1 and "--min-decode-tps" in capsys.readouterr().err
    # a batch decodes together and counts every sequence's tokens
    m = M.EngineBench(model, batch=3).run_decode_throughput([5, 6, 7], 4)
    assert m["batch"] == 3 and m["decode_tokens"] == 4


def test_refused_steps_launch_nothing(loaded):
    """What the host can see is wrong with a step is refused before anything runs: no kernel
    is launched, no page is taken, no length moves."""
    from inference_engine_rust_b200 import StepError
    from inference_engine_rust_b200.cache import CacheFull
    from inference_engine_rust_b200.csrc import bindings as B
    folder, model, w = loaded["A"]
    eng = model.session(max_tokens=128, max_sequences=3, max_seq_len=100).engine
    a, b = eng.open_sequence(), eng.open_sequence()
    eng.step([(a, [1, 2, 3])], want=None)                      # a holds three tokens, b none
    torch.cuda.synchronize()
    vocab = TINY["A"]["vocab_size"]
    cases = [
        ([], StepError),                                       # no sequence
        ([(a, [])], StepError),                                # no tokens
        ([(a, [1]), (a, [2])], StepError),                     # a slot twice
        ([(a, [vocab])], StepError), ([(b, [-1])], StepError),  # ids outside the vocabulary
        ([(a, [1, 2])], StepError),                            # several tokens into a sequence that has begun
        ([(a, [1]), (b, [1, 2])], StepError),                  # one goes on, one starts
        ([(2, [1])], StepError),                               # a slot nobody holds
        ([(b, [1] * 101)], CacheFull),                         # longer than the cache's longest sequence
        ([(a, [1])], StepError, [[1]]),                        # a wanted place outside the tokens
    ]
    launches, pages, replayed = B.launch_count, eng.cache.kv_groups[0].pages.free_count, eng.graph_launches
    for case in cases:
        entries, exc = case[0], case[1]
        want = case[2] if len(case) > 2 else "last"
        with pytest.raises(exc):
            eng.step(entries, want=want)
        assert B.launch_count == launches and eng.graph_launches == replayed
        assert eng.cache.kv_groups[0].pages.free_count == pages
        assert eng.length(a) == 3 and eng.length(b) == 0
    eng.check_device()
    # a cache without a free page: the step is refused when it asks for room, nothing has run
    small = model.session(max_tokens=64, max_sequences=2).engine
    s1, s2 = small.open_sequence(), small.open_sequence()
    small.step([(s1, [1, 2])], want=None)
    launches = B.launch_count
    with pytest.raises(CacheFull):
        small.step([(s2, [3])], want=None)
    assert B.launch_count == launches
