"""The engine against the plain implementation on the tiny configurations, in 32-bit and in
bfloat16, under every way of cutting the work: each request alone and whole; with its last
32 tokens one by one; in batches of unequal lengths whose shorter requests end earlier, one
batch after another through the same few slots."""
import functools

import pytest
import torch

from helpers import TINY, compare, make_folder, plain_weights, prompts_for
from plain import mistral_plain as P

pytestmark = pytest.mark.gpu

LENGTHS = {
    "A": [5, 11, 23, 70, 150],        # window 16, ring of 64 positions: 70 and 150 wrap it
    "B": [1, 7, 19, 40, 130],
    "C": [3, 64, 65, 129, 200],       # window 70, ring of 128 positions
    "D": [2, 9, 41, 66, 90],          # sizes only the plain kernels take
}
CASES = [(c, d) for c in ("A", "B", "C", "D") for d in ("float32", "bfloat16")]


@functools.lru_cache(maxsize=None)
def _setup(tmp_root, name, dtype):
    from inference_engine_rust_b200 import LoadedModel
    cfg = TINY[name]
    folder = make_folder(tmp_root, cfg, seed=11, dtype=dtype)
    model = LoadedModel.load(folder, dtype=dtype)
    weights = plain_weights(folder)
    prompts = prompts_for(cfg, LENGTHS[name], seed=5)
    rnd = P.bf16_rounding if dtype == "bfloat16" else P.no_rounding
    want = [P.forward(cfg, weights, p, rnd) for p in prompts]
    return model, prompts, want


@pytest.fixture(scope="module")
def tmp_root(tmp_path_factory):
    return str(tmp_path_factory.mktemp("models"))


def new_engine(model, max_tokens=64 * 12, **kw):
    return model.session(max_tokens=max_tokens, poison_cache=True, **kw).engine


@pytest.mark.parametrize("name,dtype", CASES)
def test_each_request_alone_and_whole(tmp_root, name, dtype):
    model, prompts, want = _setup(tmp_root, name, dtype)
    eng = new_engine(model)
    for i, (p, ref) in enumerate(zip(prompts, want)):
        slot = eng.open_sequence()
        got = eng.step([(slot, p)], want="all")
        eng.check_device()
        compare(got, ref, dtype, f"{name} request {i} ({len(p)} tokens) whole")
        eng.close_sequence(slot)
    eng.cache.check()


@pytest.mark.parametrize("name,dtype", CASES)
def test_last_tokens_one_by_one(tmp_root, name, dtype):
    model, prompts, want = _setup(tmp_root, name, dtype)
    eng = new_engine(model)
    for i, (p, ref) in enumerate(zip(prompts, want)):
        tail = min(32, len(p) - 1)
        head = len(p) - tail
        slot = eng.open_sequence()
        rows = [eng.step([(slot, p[:head])], want="all")]
        for t in p[head:]:
            rows.append(eng.step([(slot, [t])], want="last"))
        eng.check_device()
        got = torch.cat(rows)
        compare(got[:head], ref[:head], dtype, f"{name} request {i}: prompt part")
        compare(got[head:], ref[head:], dtype, f"{name} request {i}: {tail} tokens decoded one by one")
        assert eng.length(slot) == len(p)
        eng.close_sequence(slot)


@pytest.mark.parametrize("name,dtype", CASES)
def test_unequal_batches_through_reused_slots(tmp_root, name, dtype):
    """Batches of 2 and 3 requests in a cache with 3 slots; each request's prompt is all but
    its last d tokens with a different d per request, so requests leave the batch one
    after another while the others go on."""
    model, prompts, want = _setup(tmp_root, name, dtype)
    eng = new_engine(model, max_tokens=64 * 9, max_sequences=3)
    order = [[4, 0], [3, 1, 2]] if name != "B" else [[4, 1], [3, 0, 2]]
    used_slots = []
    for batch in order:
        slots = {i: eng.open_sequence() for i in batch}
        used_slots.append(sorted(slots.values()))
        tails = {i: min(len(prompts[i]) - 1, 3 + 4 * k) for k, i in enumerate(batch)}
        got = {i: [] for i in batch}
        out = eng.step([(slots[i], prompts[i][:len(prompts[i]) - tails[i]]) for i in batch], want="all")
        at = 0
        for i in batch:
            n = len(prompts[i]) - tails[i]
            got[i].append(out[at:at + n])
            at += n
        live = [i for i in batch if tails[i] > 0]
        for i in batch:
            if tails[i] == 0:
                eng.close_sequence(slots[i])
        k = 0
        while live:
            entries = [(slots[i], [prompts[i][len(prompts[i]) - tails[i] + k]]) for i in live]
            out = eng.step(entries, want="last")
            for r, i in enumerate(live):
                got[i].append(out[r:r + 1])
            k += 1
            for i in [i for i in live if tails[i] == k]:
                eng.close_sequence(slots[i])
            live = [i for i in live if tails[i] > k]
        eng.check_device()
        eng.cache.check()
        for i in batch:
            compare(torch.cat(got[i]), want[i], dtype, f"{name} request {i} in batch {batch}")
    assert used_slots[0][0] in used_slots[1], "the second batch did not reuse a slot"
    assert eng.cache.slots.free_count == 3


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "bfloat16")])
def test_wanted_places_and_padding_free_packing(tmp_root, name, dtype):
    """Logits only where wanted, in the order of the entries and of `want`; a request's logits
    do not depend on which other requests share the step."""
    model, prompts, want = _setup(tmp_root, name, dtype)
    eng = new_engine(model)
    batch = [1, 3, 2]
    places = {1: [0, len(prompts[1]) - 1], 3: [], 2: [2, 1]}
    slots = {i: eng.open_sequence() for i in batch}
    out = eng.step([(slots[i], prompts[i]) for i in batch], want=[places[i] for i in batch])
    eng.check_device()
    ref = torch.stack([want[1][0], want[1][-1], want[2][2], want[2][1]])
    compare(out, ref, dtype, "wanted places")
    assert eng.step([(slots[1], [7])], want=None) is None
    for i in batch:
        eng.close_sequence(slots[i])


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("A", "bfloat16"), ("B", "float32")])
def test_long_decoding_and_first_tokens(tmp_root, name, dtype):
    """A sequence decoded from its very first token, one token a step, far past the window
    and over several pages."""
    from inference_engine_rust_b200 import LoadedModel
    cfg = TINY[name]
    folder = make_folder(tmp_root, cfg, seed=11, dtype=dtype)
    model, _, _ = _setup(tmp_root, name, dtype)
    ids = prompts_for(cfg, [210], seed=9)[0]
    rnd = P.bf16_rounding if dtype == "bfloat16" else P.no_rounding
    ref = P.forward(cfg, plain_weights(folder), ids, rnd)
    eng = new_engine(model)
    slot = eng.open_sequence()
    rows = [eng.step([(slot, [t])], want="last") for t in ids]
    eng.check_device()
    got = torch.cat(rows)
    compare(got[:4], ref[:4], dtype, f"{name}: the first tokens of a sequence")
    compare(got, ref, dtype, f"{name}: 210 tokens decoded one by one")


ODD = {
    # head_dim beyond what the tensor-core attention kernels take (plain kernels), with a window
    "head_dim_272": dict(num_hidden_layers=1, hidden_size=128, num_attention_heads=3, num_key_value_heads=3, head_dim=272,
                         intermediate_size=64, vocab_size=1001, sliding_window=50),
    # one head, a window of one position (every token sees only itself), a vocabulary of three
    "one_head_window_1": dict(num_hidden_layers=2, hidden_size=48, num_attention_heads=1, num_key_value_heads=1, head_dim=48,
                              intermediate_size=8, vocab_size=3, sliding_window=1),
    # sixteen query heads per kv head: two slices of the decode kernel's 8-row tile
    "group_of_16": dict(num_hidden_layers=1, hidden_size=256, num_attention_heads=32, num_key_value_heads=2, head_dim=16,
                        intermediate_size=72, vocab_size=515, sliding_window=None),
    # the smallest head there is
    "head_dim_2": dict(num_hidden_layers=1, hidden_size=24, num_attention_heads=6, num_key_value_heads=3, head_dim=2,
                       intermediate_size=40, vocab_size=50, sliding_window=None),
}


@pytest.mark.parametrize("name", sorted(ODD))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_at_the_edges(tmp_root, name, dtype):
    """Sizes at the edge of what the kernels take: each either runs on a kernel that takes it or
    falls back to the plain one; never a wrong result."""
    from inference_engine_rust_b200 import LoadedModel
    cfg = dict(TINY["A"], **ODD[name])
    folder = make_folder(tmp_root, cfg, seed=2, dtype=dtype)
    model = LoadedModel.load(folder, dtype=dtype)
    w = plain_weights(folder)
    rnd = P.bf16_rounding if dtype == "bfloat16" else P.no_rounding
    eng = new_engine(model, max_tokens=64 * 8)
    for n in (1, 70, 130):
        p = prompts_for(cfg, [n], seed=n)[0]
        ref = P.forward(cfg, w, p, rnd)
        s = eng.open_sequence()
        head = max(1, n - 5)
        rows = [eng.step([(s, p[:head])], want="all")] + [eng.step([(s, [t])], want="last") for t in p[head:]]
        eng.check_device()
        compare(torch.cat(rows), ref, dtype, f"{name} {dtype}, {n} tokens")
        eng.close_sequence(s)


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("A", "bfloat16"), ("C", "bfloat16"), ("B", "float32")])
def test_short_prompts_through_captured_graphs(tmp_root, name, dtype):
    """Short prompt steps replay a captured graph from the second use of a shape bucket on (tokens
    padded to 16, 32 or a multiple of 64, sequences to a power of two).  Padding changes no result: the
    logits equal those of the same step launched kernel by kernel, and the cache holds the same."""
    model, prompts, want = _setup(tmp_root, name, dtype)
    cfg = TINY[name]
    eager = new_engine(model, max_tokens=64 * 24, use_graphs=False)
    graph = new_engine(model, max_tokens=64 * 24)
    assert graph.use_graphs
    sets = [prompts_for(cfg, lens, seed=40 + k) for k, lens in enumerate(
        ([1], [16], [17], [33], [63], [64], [65], [5, 11, 23], [2, 3], [130, 7, 60], [3, 1, 2, 9, 17], [200, 250]))]
    for rep in range(3):                       # first use of a bucket: eager; from the second on: replay
        for ps in sets:
            out = {}
            for label, eng in (("eager", eager), ("graph", graph)):
                slots = [eng.open_sequence() for _ in ps]
                first = eng.step(list(zip(slots, ps)), want="last")
                nxt = eng.step([(s, [7 % cfg["vocab_size"]]) for s in slots], want="last")   # reads the cache the prompt wrote
                eng.check_device()
                out[label] = torch.cat([first, nxt]).clone()
                for s in slots:
                    eng.close_sequence(s)
            compare(out["graph"], out["eager"], dtype, f"{name} {dtype} prompts of {[len(p) for p in ps]}, pass {rep}")
            if dtype == "float32":
                assert torch.equal(out["graph"], out["eager"]), "the true 32-bit path must not depend on padding at all"
    assert any(isinstance(k, tuple) and k[0] == "prompt" for k in graph._graphs), "no prompt graph was captured"
    assert graph.graph_launches > 0
