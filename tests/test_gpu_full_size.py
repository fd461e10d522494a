"""The engine at Mistral-7B layer sizes (hidden 4096, 32 heads / 8 kv heads of 128, feed-forward
14336, vocabulary 32000; two layers so that it stays small): the kernels run the shapes they
run in production (k of 4096 and 14336, split-K, 128-wide heads, four query heads per kv
head).

  * the plain implementation on the CPU, on the same weights (made on the device, copied back),
    for the 37-token and the 300-token request: the engine's float32 path against it at the
    float32 tolerance, the bfloat16 engine (tcgen05 projections and prompt attention, TMA decode
    attention) against the plain implementation with bfloat16 rounding;
  * float32: the logits of a request do not depend on how its tokens are cut into steps or on
    what else is in the batch;
  * bfloat16 (tensor-core kernels) against float32 on the same bf16-rounded weights.

The reference's like checks: logits of a prompt against an independent implementation with
difference statistics (tests/prefill_smoke.rs:99-143, tests/common/llama_logits_helpers.rs:16-89).
"""
import pytest
import torch

from helpers import compare
from plain import mistral_plain as P

pytestmark = pytest.mark.gpu

CFG = {
    "architectures": ["MistralForCausalLM"], "model_type": "mistral",
    "num_hidden_layers": 2, "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 128, "intermediate_size": 14336, "vocab_size": 32000, "rope_theta": 10000.0,
    "sliding_window": 160, "rms_norm_eps": 1e-5, "max_position_embeddings": 4096,
    "tie_word_embeddings": False, "hidden_act": "silu", "bos_token_id": 1, "eos_token_id": 2,
}
LENGTHS = [300, 37, 129]          # the window of 160 cuts the longest request; 300 > two pages


@pytest.fixture(scope="module")
def models():
    from inference_engine_rust_b200 import LoadedModel
    from inference_engine_rust_b200.weights import RandomSource
    bf = LoadedModel.random(CFG, seed=5, dtype="bfloat16", std=0.02, on_device=True)
    # the float32 model gets the very same (bf16-rounded) numbers, widened
    f32 = LoadedModel._build(bf.config, "float32", "cuda:0", False)
    src = RandomSource(f32.expected_tensors(), 5, 0.02, dtype=torch.bfloat16, device="cuda:0")
    f32.load(src, where="random weights")
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, CFG["vocab_size"], (n,), generator=g).tolist() for n in LENGTHS]
    return bf, LoadedModel(bf.config, f32), prompts


@pytest.fixture(scope="module")
def plain_logits(models):
    """Logits of the plain implementation for requests 1 (37 tokens) and 0 (300 tokens: the window
    of 160 binds), without rounding and with the rounding of a bfloat16 engine."""
    from inference_engine_rust_b200.weights import RandomSource
    bf, f32, prompts = models
    src = RandomSource(f32.model.expected_tensors(), 5, 0.02, dtype=torch.bfloat16, device="cuda:0")
    w = {name: src.get(name).float().cpu() for name in src.names()}
    out = {}
    for i in (1, 0):
        out[i] = (P.forward(CFG, w, prompts[i], P.no_rounding), P.forward(CFG, w, prompts[i], P.bf16_rounding))
    return out


def run_whole(model, prompts):
    eng = model.session(max_tokens=64 * 12, poison_cache=True).engine
    out = []
    for p in prompts:
        s = eng.open_sequence()
        out.append(eng.step([(s, p)], want="all").clone())
        eng.close_sequence(s)
    eng.check_device()
    return out


def run_batched_with_tails(model, prompts, tails):
    """All prompts (minus their tails) in one step, then one token each until each ends."""
    eng = model.session(max_tokens=64 * 12, max_sequences=4, poison_cache=True).engine
    slots = [eng.open_sequence() for _ in prompts]
    got = [[] for _ in prompts]
    out = eng.step([(s, p[:len(p) - t]) for s, p, t in zip(slots, prompts, tails)], want="all")
    at = 0
    for i, (p, t) in enumerate(zip(prompts, tails)):
        got[i].append(out[at:at + len(p) - t].clone())
        at += len(p) - t
    for k in range(max(tails)):
        live = [i for i in range(len(prompts)) if tails[i] > k]
        out = eng.step([(slots[i], [prompts[i][len(prompts[i]) - tails[i] + k]]) for i in live], want="last")
        for r, i in enumerate(live):
            got[i].append(out[r:r + 1].clone())
        for i in live:
            if tails[i] == k + 1:
                eng.close_sequence(slots[i])
    eng.check_device()
    eng.cache.check()
    return [torch.cat(g) for g in got]


def test_float32_matches_the_plain_implementation(models, plain_logits):
    bf, f32, prompts = models
    whole = run_whole(f32, prompts)
    for i, (exact, _) in plain_logits.items():
        compare(whole[i], exact, "float32", f"7B sizes, float32 whole against the plain implementation, request {i}")
    cut = run_batched_with_tails(f32, prompts, tails=[32, 5, 17])
    for i, (exact, _) in plain_logits.items():
        compare(cut[i], exact, "float32", f"7B sizes, float32 batched and decoded against the plain implementation, request {i}")


def test_bfloat16_matches_the_plain_implementation(models, plain_logits):
    bf, f32, prompts = models
    whole = run_whole(bf, prompts)
    cut = run_batched_with_tails(bf, prompts, tails=[32, 5, 17])
    for i, (_, rounded) in plain_logits.items():
        compare(whole[i], rounded, "bfloat16", f"7B sizes, bfloat16 whole against the plain implementation, request {i}")
        compare(cut[i], rounded, "bfloat16", f"7B sizes, bfloat16 batched and decoded against the plain implementation, request {i}")


def test_float32_does_not_depend_on_the_cutting(models):
    bf, f32, prompts = models
    whole = run_whole(f32, prompts)
    cut = run_batched_with_tails(f32, prompts, tails=[32, 5, 17])
    for i, (a, b) in enumerate(zip(cut, whole)):
        compare(a, b, "float32", f"7B sizes, float32, request {i}: batched and decoded against whole")


def test_bfloat16_matches_float32(models):
    bf, f32, prompts = models
    want = run_whole(f32, prompts)
    whole = run_whole(bf, prompts)
    for i, (a, b) in enumerate(zip(whole, want)):
        compare(a, b, "bfloat16", f"7B sizes, bfloat16 whole against float32, request {i}")
    cut = run_batched_with_tails(bf, prompts, tails=[32, 5, 17])
    for i, (a, b) in enumerate(zip(cut, want)):
        compare(a, b, "bfloat16", f"7B sizes, bfloat16 batched and decoded against float32, request {i}")


def test_bfloat16_runs_are_bitwise_repeatable(models):
    """No kernel adds in an order that depends on timing (split-K partial tiles and attention
    splits are merged in a fixed order whichever CTA finishes last): the same requests give
    the same bits, whole and batched with decoding, on fresh sessions."""
    bf, f32, prompts = models
    a = run_batched_with_tails(bf, prompts, tails=[32, 5, 17])
    b = run_batched_with_tails(bf, prompts, tails=[32, 5, 17])
    for i, (x, y) in enumerate(zip(a, b)):
        assert torch.equal(x, y), f"request {i}: two identical runs differ"
    w1, w2 = run_whole(bf, prompts), run_whole(bf, prompts)
    for i, (x, y) in enumerate(zip(w1, w2)):
        assert torch.equal(x, y), f"request {i}: two identical prompt runs differ"


def test_a_prompt_of_2400_tokens_then_three_tokens(models):
    """2,400 tokens in one step: the down projection's activations (2,400 x 14,336) exceed 64 MB, so
    its token tiles are walked in groups, the residual adds go through TMA, and the prompt spans 38
    pages; then three tokens one by one.  bfloat16 against the float32 path at chosen places."""
    bf, f32, prompts = models
    g = torch.Generator().manual_seed(17)
    prompt = torch.randint(0, CFG["vocab_size"], (2400,), generator=g).tolist()
    tail = torch.randint(0, CFG["vocab_size"], (3,), generator=g).tolist()
    places = [0, 1, 63, 64, 127, 128, 255, 256, 1023, 1024, 2047, 2399]
    out = {}
    for name, model in (("float32", f32), ("bfloat16", bf)):
        eng = model.session(max_tokens=64 * 40, max_sequences=1, poison_cache=True).engine
        s = eng.open_sequence()
        rows = [eng.step([(s, prompt)], want=[places]).clone()]
        for t in tail:
            rows.append(eng.step([(s, [t])], want="last").clone())
        eng.check_device()
        eng.close_sequence(s)
        eng.cache.check()
        out[name] = torch.cat(rows)
    compare(out["bfloat16"], out["float32"], "bfloat16", "7B sizes, 2,400-token prompt and three tokens")
