"""Each part of a layer alone against the plain implementation, and the generality of the
assembly: a toy mixer with state of its own, defined here, is registered, built and stepped
without a change to the package; a layer is run twice; a layer reads another layer's
cache; layers of one model use different mixers, feed-forwards (one with routing) and position
encodings."""
import math
from dataclasses import dataclass

import pytest
import torch

from helpers import compare
from plain import mistral_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def runtime(dtype=torch.float32):
    from inference_engine_rust_b200.parts.base import Runtime
    return Runtime(dtype=dtype, device=DEV)


def context(rt, q_lens, pos0, slots, kind):
    """A StepContext over explicit sequences (what Engine.step builds from its entries)."""
    import numpy as np
    from inference_engine_rust_b200.csrc import bindings as B
    from inference_engine_rust_b200.parts.base import StepContext
    n, T = len(q_lens), sum(q_lens)
    cu = np.zeros(n + 1, dtype=np.int32)
    cu[1:] = np.cumsum(q_lens)
    arrs = [torch.tensor(a, dtype=torch.int32, device=DEV) for a in
            (cu, slots, np.repeat(np.arange(n, dtype=np.int32), q_lens), pos0)]
    view = B.BatchView(cu_q=arrs[0].data_ptr(), slot_ids=arrs[1].data_ptr(), tok_seq=arrs[2].data_ptr(),
                       pos0=arrs[3].data_ptr(), n_seqs=n, n_tokens=T)
    ctx = StepContext(kind=kind, batch=view, n_tokens=T, n_seqs=n, q_lens=list(q_lens), pos0=list(pos0),
                      slots=list(slots), stream=B.stream_ptr(), rt=rt, slot_ids_dev=arrs[1], pos0_dev=arrs[3],
                      cu_q_dev=arrs[0])
    ctx._keep = arrs
    return ctx


def spec(kind, **params):
    from inference_engine_rust_b200.config.specs import PartSpec
    return PartSpec(kind, params)


# ---------------------------------------------------------------------------------------
# parts alone


def test_norm_part():
    from inference_engine_rust_b200.parts import part_class
    rt = runtime()
    norm = part_class("norm", "rmsnorm")(spec("rmsnorm", eps=3e-4), 88, rt)
    assert norm.tensor_specs()["weight"].shape == (88,)
    w = torch.rand(88) + 0.5
    norm.load({"weight": w.to(DEV)})
    x = torch.randn(6, 88) * 2
    out = torch.empty(6, 88, device=DEV)
    norm.forward(x.to(DEV), out, context(rt, [6], [0], [0], "prompt"))
    compare(out, P.rmsnorm(x, w, 3e-4), "float32", "rmsnorm part")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_feed_forward_part(dtype):
    from inference_engine_rust_b200.parts import part_class
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    rt = runtime(tdt)
    ffn = part_class("ffn", "swiglu")(spec("swiglu", hidden_size=88, intermediate_size=200), rt)
    torch.manual_seed(0)
    w = {n: (torch.randn(s.shape) * 0.1).to(tdt) for n, s in ffn.tensor_specs().items()}
    ffn.load({n: t.to(DEV) for n, t in w.items()})
    x = torch.randn(9, 88).to(tdt)
    res = torch.randn(9, 88)
    res_dev = res.to(DEV)
    ffn.forward(x.to(DEV), res_dev, context(rt, [9], [0], [0], "prompt"))
    rnd = P.bf16_rounding if dtype == "bfloat16" else P.no_rounding
    ref = res + P.ffn_layer(x.float(), w["gate_proj.weight"].float(), w["up_proj.weight"].float(),
                            w["down_proj.weight"].float(), rnd)
    compare(res_dev, ref, dtype, "swiglu part adds into the residual")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kvh,hd,window,pairing,rotary", [
    (4, 2, 16, 16, "half", 16), (6, 1, 32, None, "interleaved", 32), (3, 3, 48, 70, "half", 32)])
def test_attention_part_prompt_then_decode(dtype, heads, kvh, hd, window, pairing, rotary):
    """The mixer alone: two prompts of unequal lengths in one step, then three single tokens
    each, against the plain attention of the whole sequences."""
    from inference_engine_rust_b200.cache import Cache
    from inference_engine_rust_b200.parts import part_class
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    rt = runtime(tdt)
    H, theta = 72, 5000.0
    pos = spec("rope", theta=theta, rotary_dim=rotary, pairing=pairing)
    attn = part_class("mixer", "attention")(
        spec("attention", hidden_size=H, heads=heads, kv_heads=kvh, head_dim=hd, window=window,
             scale=1 / math.sqrt(hd), position=pos), rt)
    torch.manual_seed(1)
    w = {n: (torch.randn(s.shape) * 0.15).to(tdt) for n, s in attn.tensor_specs().items()}
    attn.load({n: t.to(DEV) for n, t in w.items()})
    cache = Cache({0: attn.cache_request()}, max_tokens=64 * 8, max_seq_len=512, max_sequences=2,
                  dtype=tdt, device=DEV, poison=True)
    lens, extra = [90, 7], 3
    xs = [torch.randn(n + extra, H).to(tdt) for n in lens]
    rnd = P.bf16_rounding if dtype == "bfloat16" else P.no_rounding
    refs = [P.attention_layer(x.float(), *(w[k + "_proj.weight"].float() for k in "qkvo"), heads=heads,
                              kv_heads=kvh, head_dim=hd, rope_theta=theta, window=window, pairing=pairing,
                              rotary_dim=rotary, rnd=rnd) for x in xs]
    slots = [cache.open_sequence() for _ in lens]
    for s, n in zip(slots, lens):
        cache.reserve(s, n + extra)
    cache.upload()
    xn = torch.cat([x[:n] for x, n in zip(xs, lens)]).to(DEV)
    res = torch.zeros(sum(lens), H, device=DEV)
    attn.forward(xn, res, context(rt, lens, [0, 0], slots, "prompt"), cache.layer_view(0), True)
    compare(res, torch.cat([r[:n] for r, n in zip(refs, lens)]), dtype, "attention part, prompts")
    for k in range(extra):
        xn = torch.stack([x[n + k] for x, n in zip(xs, lens)]).to(DEV)
        res = torch.zeros(2, H, device=DEV)
        attn.forward(xn, res, context(rt, [1, 1], [n + k for n in lens], slots, "decode"), cache.layer_view(0), True)
        compare(res, torch.stack([r[n + k] for r, n in zip(refs, lens)]), dtype, f"attention part, decode {k}")
    assert rt.err.item() == 0


def test_rope_part_constants():
    from inference_engine_rust_b200.parts import part_class
    rt = runtime()
    rope = part_class("position", "rope")(spec("rope", theta=1e6, rotary_dim=32, pairing="half"), 32, rt)
    want = torch.tensor([1e6 ** (-2 * k / 32) for k in range(16)], dtype=torch.float64).float()
    assert torch.equal(rope.inv_freq.cpu(), want)
    scaled = part_class("position", "rope")(spec("rope", theta=1e6, rotary_dim=32, pairing="interleaved",
                                                 freq_factors=[2.0] * 16), 32, rt)
    assert torch.allclose(scaled.inv_freq.cpu(), want / 2) and scaled.pairing != rope.pairing
    for bad in (dict(rotary_dim=34), dict(rotary_dim=15), dict(pairing="odd")):
        with pytest.raises(ValueError):
            part_class("position", "rope")(spec("rope", **{"theta": 1e4, "rotary_dim": 32, "pairing": "half", **bad}), 32, rt)


# ---------------------------------------------------------------------------------------
# a toy architecture, defined here: layer 0 = attention, layer 1 = a mixer with state of its
# own (running mean of its inputs over the sequence, then a projection)


class RunningMeanMixer:
    """y_t = W . mean(x_0 .. x_t).  Its per-sequence state is the running sum [hidden]."""

    def __init__(self, part_spec, rt):
        from inference_engine_rust_b200.parts.linear import Linear
        self.rt, self.hidden = rt, int(part_spec["hidden_size"])
        self.Linear = Linear
        self.proj = None

    def tensor_specs(self):
        from inference_engine_rust_b200.weights import TensorSpec
        return {"proj.weight": TensorSpec((self.hidden, self.hidden))}

    def load(self, tensors):
        self.proj = self.Linear(tensors["proj.weight"], self.rt)

    def cache_request(self):
        from inference_engine_rust_b200.cache import StateRequest
        return StateRequest((self.hidden,), torch.float32)

    def weight_bytes(self):
        return self.proj.nbytes()

    def forward(self, xn, residual, ctx, cache_view, writes_cache):
        state = cache_view.state                       # [n_slots, hidden]
        means = torch.empty(ctx.n_tokens, self.hidden, device=xn.device, dtype=torch.float32)
        t = 0
        for slot, p0, q in zip(ctx.slots, ctx.pos0, ctx.q_lens):
            sums = state[slot] + torch.cumsum(xn[t:t + q].float(), dim=0)
            counts = torch.arange(p0 + 1, p0 + q + 1, device=xn.device, dtype=torch.float32)
            means[t:t + q] = sums / counts[:, None]
            state[slot] = sums[-1]
            t += q
        self.proj.apply(means.to(self.rt.dtype), residual, ctx.n_tokens, ctx.stream, add_residual=True)


@dataclass(frozen=True)
class ToyConfig:
    hidden_size: int
    vocab_size: int
    schedule: tuple            # ((layer, reads_cache_of), ...)
    architecture: str = "ToyForCausalLM"

    @classmethod
    def from_dict(cls, raw):
        return cls(raw["hidden_size"], raw["vocab_size"], tuple(tuple(e) for e in raw["schedule"]))


def toy_spec(cfg: ToyConfig):
    from inference_engine_rust_b200.config.specs import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    H = cfg.hidden_size
    norm = PartSpec("rmsnorm", {"eps": 1e-5})
    attn = PartSpec("attention", {"hidden_size": H, "heads": 4, "kv_heads": 2, "head_dim": 16, "window": None,
                                  "scale": 0.25, "position": PartSpec("rope", {"theta": 1e4, "rotary_dim": 16, "pairing": "half"})})
    mean = PartSpec("running_mean", {"hidden_size": H})
    ffn = PartSpec("swiglu", {"hidden_size": H, "intermediate_size": 96})
    layers = []
    for i, mixer in enumerate((attn, mean, attn)):
        p = f"toy.{i}."
        layers.append(LayerSpec(block=PartSpec("prenorm", {}), norm=norm, mixer=mixer, ffn=ffn, mixer_prefix=p + "mix.",
                                ffn_prefix=p + "ffn.", mixer_norm_name=p + "n1.weight", ffn_norm_name=p + "n2.weight"))
    return ModelSpec(architecture=cfg.architecture, hidden_size=H, vocab_size=cfg.vocab_size, layers=tuple(layers),
                     schedule=tuple(ScheduleEntry(l, r) for l, r in cfg.schedule), final_norm=norm,
                     embedding_name="toy.embed.weight", final_norm_name="toy.norm.weight", lm_head_name=None,
                     embedding_scale=2.0, max_position=256, bos_token_id=None, eos_token_id=None)


@pytest.fixture(scope="module")
def toy_registered():
    from inference_engine_rust_b200.config import registry
    from inference_engine_rust_b200.parts import register_part, unregister_part
    register_part("mixer", "running_mean", RunningMeanMixer)
    registry.register_architecture("ToyForCausalLM", ToyConfig, toy_spec)
    yield
    unregister_part("mixer", "running_mean")
    registry._ARCHITECTURES.pop("ToyForCausalLM", None)


def plain_toy(cfg: ToyConfig, w, ids):
    """The toy model, whole sequence, from the plain parts."""
    x = P.embed(w["toy.embed.weight"], ids, 2.0)
    kv = {}
    for pos, (layer, reads) in enumerate(cfg.schedule):
        p = f"toy.{layer}."
        xn = P.rmsnorm(x, w[p + "n1.weight"], 1e-5)
        if layer == 1:
            mean = torch.cumsum(xn, 0) / torch.arange(1, len(ids) + 1)[:, None]
            x = x + P.matmul(mean, w[p + "mix.proj.weight"])
        else:
            a = dict(heads=4, kv_heads=2, head_dim=16, rope_theta=1e4, window=None, scale=0.25)
            y, parts = P.attention_layer(xn, *(w[p + f"mix.{k}_proj.weight"] for k in "qkvo"), return_parts=True, **a)
            if reads is None:
                kv[pos] = parts
            else:                      # queries of this layer over the keys and values of entry `reads`
                q, src, T = parts["q"], kv[reads], len(ids)
                out = torch.zeros(T, 4, 16)
                mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
                for h in range(4):
                    s = (q[:, h] @ src["k"][:, h // 2].t()) * 0.25
                    out[:, h] = P.softmax(s.masked_fill(~mask, float("-inf"))) @ src["v"][:, h // 2]
                y = P.matmul(out.reshape(T, 64), w[p + "mix.o_proj.weight"])
            x = x + y
        xn = P.rmsnorm(x, w[p + "n2.weight"], 1e-5)
        x = x + P.ffn_layer(xn, w[p + "ffn.gate_proj.weight"], w[p + "ffn.up_proj.weight"], w[p + "ffn.down_proj.weight"])
    return P.matmul(P.rmsnorm(x, w["toy.norm.weight"], 1e-5), w["toy.embed.weight"])


@pytest.mark.parametrize("schedule", [
    ((0, None), (1, None)),                          # attention, then the stateful toy mixer
    ((0, None), (1, None), (0, None), (1, None)),    # both layers run twice, each run with a cache of its own
    ((0, None), (1, None), (2, 0)),                  # layer 2 reads the cache that entry 0 wrote
])
def test_toy_architecture_is_registered_built_and_stepped(toy_registered, schedule):
    from inference_engine_rust_b200 import LoadedModel
    from inference_engine_rust_b200.weights import RandomSource
    raw = {"architectures": ["ToyForCausalLM"], "hidden_size": 64, "vocab_size": 97, "schedule": [list(e) for e in schedule]}
    model = LoadedModel.random(raw, seed=4, dtype="float32", std=0.1)
    cfg = model.config
    src = RandomSource(model.model.expected_tensors(), 4, 0.1, dtype=torch.float32)
    w = {n: src.get(n) for n in src.names()}
    used = {e[0] for e in schedule}
    assert ("toy.1.mix.proj.weight" in w) and ("toy.0.mix.q_proj.weight" in w)
    eng = model.session(max_tokens=64 * 6, poison_cache=True).engine
    kinds = sorted(type(g).__name__ for g in eng.cache.kv_groups + eng.cache.state_groups)
    assert kinds == ["KVGroup", "StateGroup"]
    n_kv = sum(1 for l, r in schedule if l != 1 and r is None)
    assert sum(len(g.layers) for g in eng.cache.kv_groups) == n_kv
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 97, (n,), generator=g).tolist() for n in (37, 5, 70)]
    want = [plain_toy(cfg, w, p) for p in prompts]
    # whole; then in a batch with the last tokens one by one; slots are used again in between
    for p, ref in zip(prompts, want):
        s = eng.open_sequence()
        compare(eng.step([(s, p)], want="all"), ref, "float32", "toy model, whole")
        eng.close_sequence(s)
    slots = [eng.open_sequence() for _ in prompts]
    tails = [4, 2, 6]
    got = [[] for _ in prompts]
    out = eng.step([(s, p[:len(p) - t]) for s, p, t in zip(slots, prompts, tails)], want="all")
    at = 0
    for i, (p, t) in enumerate(zip(prompts, tails)):
        got[i].append(out[at:at + len(p) - t])
        at += len(p) - t
    for k in range(max(tails)):
        live = [i for i in range(3) if tails[i] > k]
        out = eng.step([(slots[i], [prompts[i][len(prompts[i]) - tails[i] + k]]) for i in live], want="last")
        for r, i in enumerate(live):
            got[i].append(out[r:r + 1])
    eng.check_device()
    for i in range(3):
        compare(torch.cat(got[i]), want[i], "float32", f"toy model, request {i} batched and decoded")


def test_unknown_part_kind_is_named(toy_registered):
    from inference_engine_rust_b200.parts import part_class
    with pytest.raises(KeyError) as e:
        part_class("mixer", "convolution")
    assert "attention" in str(e.value) and "running_mean" in str(e.value)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_block_part_alone(dtype):
    """The pre-norm arrangement with its four parts against the plain block, for two prompts."""
    from inference_engine_rust_b200.cache import Cache
    from inference_engine_rust_b200.config.specs import LayerSpec
    from inference_engine_rust_b200.parts import part_class
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    rt = runtime(tdt)
    H, heads, kvh, hd, I, eps = 80, 5, 5, 16, 112, 2e-5
    norm_spec = spec("rmsnorm", eps=eps)
    mixer_spec = spec("attention", hidden_size=H, heads=heads, kv_heads=kvh, head_dim=hd, window=None,
                      scale=1 / math.sqrt(hd), position=spec("rope", theta=1e4, rotary_dim=hd, pairing="half"))
    ffn_spec = spec("swiglu", hidden_size=H, intermediate_size=I)
    ls = LayerSpec(block=spec("prenorm"), norm=norm_spec, mixer=mixer_spec, ffn=ffn_spec,
                   mixer_prefix="model.layers.0.self_attn.", ffn_prefix="model.layers.0.mlp.",
                   mixer_norm_name="model.layers.0.input_layernorm.weight",
                   ffn_norm_name="model.layers.0.post_attention_layernorm.weight")
    n1 = part_class("norm", "rmsnorm")(norm_spec, H, rt)
    n2 = part_class("norm", "rmsnorm")(norm_spec, H, rt)
    mixer = part_class("mixer", "attention")(mixer_spec, rt)
    ffn = part_class("ffn", "swiglu")(ffn_spec, rt)
    block = part_class("block", "prenorm")(ls, n1, mixer, n2, ffn, rt)
    torch.manual_seed(2)
    w = {ls.mixer_norm_name: (1 + 0.1 * torch.randn(H)).to(tdt), ls.ffn_norm_name: (1 + 0.1 * torch.randn(H)).to(tdt)}
    for prefix, part in ((ls.mixer_prefix, mixer), (ls.ffn_prefix, ffn)):
        for n, s in part.tensor_specs().items():
            w[prefix + n] = (torch.randn(s.shape) * 0.15).to(tdt)
    n1.load({"weight": w[ls.mixer_norm_name].to(DEV)})
    n2.load({"weight": w[ls.ffn_norm_name].to(DEV)})
    mixer.load({n: w[ls.mixer_prefix + n].to(DEV) for n in mixer.tensor_specs()})
    ffn.load({n: w[ls.ffn_prefix + n].to(DEV) for n in ffn.tensor_specs()})
    cache = Cache({0: mixer.cache_request()}, max_tokens=64 * 4, max_seq_len=256, max_sequences=2,
                  dtype=tdt, device=DEV, poison=True)
    lens = [33, 70]
    slots = [cache.open_sequence() for _ in lens]
    for s_, n in zip(slots, lens):
        cache.reserve(s_, n)
    cache.upload()
    xs = [torch.randn(n, H) for n in lens]
    x = torch.cat(xs).to(DEV)
    block.forward(x, context(rt, lens, [0, 0], slots, "prompt"), cache.layer_view(0), True)
    cfg = {"rms_norm_eps": eps, "num_attention_heads": heads, "num_key_value_heads": kvh, "head_dim": hd,
           "rope_theta": 1e4, "sliding_window": None}
    rnd = P.bf16_rounding if dtype == "bfloat16" else P.no_rounding
    ref = torch.cat([P.block(xx, cfg, {k: v.float() for k, v in w.items()}, 0, rnd) for xx in xs])
    compare(x, ref, dtype, "pre-norm block part")


# ---------------------------------------------------------------------------------------
# two more toy parts, defined here: a feed-forward that routes each token to one of a few
# experts, and a position encoding that is no rotation


class TopOneExperts:
    """y = p_e * W2_e . relu(W1_e . x) for the expert e with the largest router logit, p being the
    softmax of the router logits (computed in 32-bit)."""

    def __init__(self, part_spec, rt):
        from inference_engine_rust_b200.parts.linear import Linear
        self.rt, self.Linear = rt, Linear
        self.hidden, self.inner, self.experts = (int(part_spec[k]) for k in ("hidden_size", "inner_size", "experts"))

    def tensor_specs(self):
        from inference_engine_rust_b200.weights import TensorSpec
        specs = {"router.weight": TensorSpec((self.experts, self.hidden))}
        for e in range(self.experts):
            specs[f"experts.{e}.w1.weight"] = TensorSpec((self.inner, self.hidden))
            specs[f"experts.{e}.w2.weight"] = TensorSpec((self.hidden, self.inner))
        return specs

    def load(self, tensors):
        self.router = tensors["router.weight"].float()
        self.w1 = [self.Linear(tensors[f"experts.{e}.w1.weight"], self.rt) for e in range(self.experts)]
        self.w2 = [self.Linear(tensors[f"experts.{e}.w2.weight"], self.rt) for e in range(self.experts)]

    def weight_bytes(self):
        return sum(l.nbytes() for l in self.w1 + self.w2)

    def forward(self, xn, residual, ctx):
        T = ctx.n_tokens
        p = torch.softmax(xn[:T].float() @ self.router.t(), dim=-1)
        top = p.argmax(dim=-1)
        for e in range(self.experts):
            idx = torch.nonzero(top == e).flatten()
            n = idx.numel()
            if n == 0:
                continue
            h = torch.empty(n, self.inner, dtype=self.rt.dtype, device=xn.device)
            self.w1[e].apply(xn[idx].contiguous(), h, n, ctx.stream)
            y = torch.zeros(n, self.hidden, dtype=torch.float32, device=xn.device)
            self.w2[e].apply(torch.relu(h), y, n, ctx.stream, add_residual=True)
            residual.index_add_(0, idx, y * p[idx, e, None])


class LearnedOffsets:
    """Queries and keys get a learned vector added that depends on the position modulo `period`;
    nothing is rotated."""

    def __init__(self, part_spec, head_dim, rt):
        self.rt, self.head_dim, self.period = rt, head_dim, int(part_spec["period"])

    def tensor_specs(self):
        from inference_engine_rust_b200.weights import TensorSpec
        return {"offsets": TensorSpec((self.period, self.head_dim))}

    def load(self, tensors):
        self.offsets = tensors["offsets"].float()

    def encode(self, qkv, ctx, heads, kv_heads):
        pos = torch.cat([torch.arange(p0, p0 + q) for p0, q in zip(ctx.pos0, ctx.q_lens)]).to(qkv.device)
        rows = qkv[:ctx.n_tokens].view(ctx.n_tokens, -1, self.head_dim)
        n = heads + kv_heads                        # queries and keys; values stay as they are
        rows[:, :n] = (rows[:, :n].float() + self.offsets[pos % self.period][:, None, :]).to(qkv.dtype)


@dataclass(frozen=True)
class RoutedToyConfig:
    hidden_size: int
    vocab_size: int
    experts: int
    period: int
    architecture: str = "RoutedToyForCausalLM"

    @classmethod
    def from_dict(cls, raw):
        return cls(raw["hidden_size"], raw["vocab_size"], raw["experts"], raw["period"])


R_HEADS, R_KV, R_HD, R_INNER = 3, 1, 32, 40


def routed_toy_spec(cfg: RoutedToyConfig):
    from inference_engine_rust_b200.config.specs import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    H = cfg.hidden_size
    norm = PartSpec("rmsnorm", {"eps": 1e-5})

    def attn(position):
        return PartSpec("attention", {"hidden_size": H, "heads": R_HEADS, "kv_heads": R_KV, "head_dim": R_HD,
                                      "window": None, "scale": R_HD ** -0.5, "position": position})
    offsets = PartSpec("learned_offsets", {"period": cfg.period})
    rope = PartSpec("rope", {"theta": 1e4, "rotary_dim": R_HD, "pairing": "half"})
    routed = PartSpec("top_one_experts", {"hidden_size": H, "inner_size": R_INNER, "experts": cfg.experts})
    dense = PartSpec("swiglu", {"hidden_size": H, "intermediate_size": 56})
    layers = []
    for i, (mixer, ffn) in enumerate(((attn(offsets), routed), (attn(rope), dense))):
        p = f"toy.{i}."
        layers.append(LayerSpec(block=PartSpec("prenorm", {}), norm=norm, mixer=mixer, ffn=ffn, mixer_prefix=p + "mix.",
                                ffn_prefix=p + "ffn.", mixer_norm_name=p + "n1.weight", ffn_norm_name=p + "n2.weight"))
    return ModelSpec(architecture=cfg.architecture, hidden_size=H, vocab_size=cfg.vocab_size, layers=tuple(layers),
                     schedule=(ScheduleEntry(0, None), ScheduleEntry(1, None)), final_norm=norm,
                     embedding_name="toy.embed.weight", final_norm_name="toy.norm.weight", lm_head_name="toy.head.weight",
                     embedding_scale=1.0, max_position=256, bos_token_id=None, eos_token_id=None)


def plain_routed_toy(cfg: RoutedToyConfig, w, ids):
    T = len(ids)
    x = P.embed(w["toy.embed.weight"], ids, 1.0)
    # layer 0: attention whose queries and keys carry learned offsets, then the routed feed-forward
    xn = P.rmsnorm(x, w["toy.0.n1.weight"], 1e-5)
    off = w["toy.0.mix.position.offsets"][torch.arange(T) % cfg.period]
    q = P.matmul(xn, w["toy.0.mix.q_proj.weight"]).view(T, R_HEADS, R_HD) + off[:, None]
    k = P.matmul(xn, w["toy.0.mix.k_proj.weight"]).view(T, R_KV, R_HD) + off[:, None]
    v = P.matmul(xn, w["toy.0.mix.v_proj.weight"]).view(T, R_KV, R_HD)
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
    out = torch.zeros(T, R_HEADS, R_HD)
    for h in range(R_HEADS):
        s = (q[:, h] @ k[:, 0].t()) * R_HD ** -0.5
        out[:, h] = P.softmax(s.masked_fill(~mask, float("-inf"))) @ v[:, 0]
    x = x + P.matmul(out.reshape(T, -1), w["toy.0.mix.o_proj.weight"])
    xn = P.rmsnorm(x, w["toy.0.n2.weight"], 1e-5)
    p = P.softmax(P.matmul(xn, w["toy.0.ffn.router.weight"]))
    y = torch.zeros_like(x)
    chosen = []
    for t in range(T):
        e = int(p[t].argmax())
        chosen.append(e)
        hcur = torch.relu(P.matmul(xn[t:t + 1], w[f"toy.0.ffn.experts.{e}.w1.weight"]))
        y[t] = p[t, e] * P.matmul(hcur, w[f"toy.0.ffn.experts.{e}.w2.weight"])[0]
    x = x + y
    # layer 1: the package's own attention with rotary positions and its dense feed-forward
    xn = P.rmsnorm(x, w["toy.1.n1.weight"], 1e-5)
    x = x + P.attention_layer(xn, *(w[f"toy.1.mix.{n}_proj.weight"] for n in "qkvo"), heads=R_HEADS, kv_heads=R_KV,
                              head_dim=R_HD, rope_theta=1e4, window=None)
    xn = P.rmsnorm(x, w["toy.1.n2.weight"], 1e-5)
    x = x + P.ffn_layer(xn, w["toy.1.ffn.gate_proj.weight"], w["toy.1.ffn.up_proj.weight"], w["toy.1.ffn.down_proj.weight"])
    return P.matmul(P.rmsnorm(x, w["toy.norm.weight"], 1e-5), w["toy.head.weight"]), chosen


def test_routed_feed_forward_and_another_position_encoding():
    """A feed-forward with routing and a position encoding that is no rotation, both defined in
    this file, in one layer of a model whose other layer uses the package's own parts."""
    from inference_engine_rust_b200 import LoadedModel
    from inference_engine_rust_b200.config import registry
    from inference_engine_rust_b200.parts import register_part, unregister_part
    from inference_engine_rust_b200.weights import RandomSource
    register_part("ffn", "top_one_experts", TopOneExperts)
    register_part("position", "learned_offsets", LearnedOffsets)
    registry.register_architecture("RoutedToyForCausalLM", RoutedToyConfig, routed_toy_spec)
    try:
        raw = {"architectures": ["RoutedToyForCausalLM"], "hidden_size": 72, "vocab_size": 113, "experts": 3, "period": 7}
        model = LoadedModel.random(raw, seed=8, dtype="float32", std=0.15)
        src = RandomSource(model.model.expected_tensors(), 8, 0.15, dtype=torch.float32)
        w = {n: src.get(n) for n in src.names()}
        assert "toy.0.mix.position.offsets" in w and "toy.0.ffn.experts.2.w2.weight" in w
        assert not any(n.startswith("toy.1.mix.position") for n in w)
        eng = model.session(max_tokens=64 * 6, poison_cache=True).engine
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(0, 113, (n,), generator=g).tolist() for n in (45, 9, 66)]
        want, chosen = zip(*(plain_routed_toy(model.config, w, p) for p in prompts))
        assert len({e for c in chosen for e in c}) == 3, "the prompts do not reach every expert"
        for p, ref in zip(prompts, want):
            s = eng.open_sequence()
            compare(eng.step([(s, p)], want="all"), ref, "float32", "routed toy, whole")
            eng.close_sequence(s)
        slots = [eng.open_sequence() for _ in prompts]
        tails = [8, 3, 5]
        got = [[] for _ in prompts]
        out = eng.step([(s, p[:len(p) - t]) for s, p, t in zip(slots, prompts, tails)], want="all")
        at = 0
        for i, (p, t) in enumerate(zip(prompts, tails)):
            got[i].append(out[at:at + len(p) - t])
            at += len(p) - t
        for k in range(max(tails)):
            live = [i for i in range(3) if tails[i] > k]
            out = eng.step([(slots[i], [prompts[i][len(prompts[i]) - tails[i] + k]]) for i in live], want="last")
            for r, i in enumerate(live):
                got[i].append(out[r:r + 1])
        eng.check_device()
        for i in range(3):
            compare(torch.cat(got[i]), want[i], "float32", f"routed toy, request {i} batched and decoded")
    finally:
        unregister_part("ffn", "top_one_experts")
        unregister_part("position", "learned_offsets")
        registry._ARCHITECTURES.pop("RoutedToyForCausalLM", None)


def test_attention_asks_for_a_cut_by_length_when_it_pays():
    """The mixer's answer to the engine's question before a one-token step: sequences of equal
    lengths keep the even cut unless the batch's CTAs leave the last round of slots mostly empty;
    one long sequence among short ones asks for the cut by length; a mixer without the method is
    not asked (the toy mixers above have none)."""
    from inference_engine_rust_b200.parts import fast_attention as FA
    from inference_engine_rust_b200.csrc import bindings as B
    slots = 2 * B.sm_count()
    assert not FA.wants_length_cut([2047] * 8, 8, 4, None, 64, 128)
    assert not FA.wants_length_cut([2047], 8, 4, None, 64, 128)
    assert FA.wants_length_cut([8191] + [1023] * 7, 8, 4, None, 64, 128)
    assert not FA.wants_length_cut([8191] + [1023] * 7, 8, 4, 1024, 64, 128), "a window makes them equal"
    full = slots // 8                                   # sequences whose CTAs fill the slots exactly
    assert not FA.wants_length_cut([2047] * full, 8, 4, None, 64, 128)
    assert FA.wants_length_cut([2047] * (full + full // 3), 8, 4, None, 64, 128), "one and a third rounds"
    assert not FA.wants_length_cut([2047] * (2 * full - 2), 8, 4, None, 64, 128), "almost two full rounds"


# ---- another block arrangement: norms after the parts too, and a layer without a feed-forward ----------


class SandwichBlock:
    """x += post_mixer(mixer(norm1(x))); x += post_ffn(ffn(norm2(x))): the two extra norms come by role
    from `LayerSpec.extra_norms`.  The parts ADD into the tensor they are given, so each gets a zeroed
    buffer, whose normed content is then added to x."""

    def __init__(self, layer_spec, norm1, mixer, norm2, ffn, rt, extra_norms=None):
        self.norm1, self.mixer, self.norm2, self.ffn, self.rt = norm1, mixer, norm2, ffn, rt
        self.post = extra_norms or {}

    def forward(self, x, ctx, cache_view, writes_cache):
        ws, T = self.rt.workspace, ctx.n_tokens
        for norm, post, run in ((self.norm1, "post_mixer", lambda xn, y: self.mixer.forward(xn, y, ctx, cache_view, writes_cache)),
                                (self.norm2, "post_ffn", (lambda xn, y: self.ffn.forward(xn, y, ctx)) if self.ffn else None)):
            if run is None:
                continue
            xn = ws.take("sandwich.normed", x.shape, self.rt.dtype)
            norm.forward(x, xn, ctx, rows=T)
            y = ws.take("sandwich.delta", x.shape, torch.float32)
            y.zero_()
            run(xn, y)
            yn = ws.take("sandwich.delta_normed", x.shape, torch.float32)
            self.post[post].forward(y, yn, ctx, rows=T)
            x[:T] += yn[:T]


@dataclass(frozen=True)
class SandwichConfig:
    hidden_size: int
    vocab_size: int
    architecture: str = "SandwichToyForCausalLM"

    @classmethod
    def from_dict(cls, raw):
        return cls(raw["hidden_size"], raw["vocab_size"])


def sandwich_spec(cfg: SandwichConfig):
    from inference_engine_rust_b200.config.specs import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    H = cfg.hidden_size
    norm = PartSpec("rmsnorm", {"eps": 1e-5})
    post = PartSpec("rmsnorm", {"eps": 1e-3})
    attn = PartSpec("attention", {"hidden_size": H, "heads": 4, "kv_heads": 2, "head_dim": 16, "window": 24,
                                  "scale": 0.25, "position": PartSpec("rope", {"theta": 1e4, "rotary_dim": 16, "pairing": "half"})})
    ffn = PartSpec("swiglu", {"hidden_size": H, "intermediate_size": 72})
    layers = []
    for i, f in enumerate((ffn, None)):          # the second layer has no feed-forward
        p = f"toy.{i}."
        extra = {"post_mixer": (post, p + "post1.weight")}
        if f is not None:
            extra["post_ffn"] = (post, p + "post2.weight")
        layers.append(LayerSpec(block=PartSpec("sandwich", {}), norm=norm, mixer=attn, ffn=f, mixer_prefix=p + "mix.",
                                ffn_prefix=p + "ffn.", mixer_norm_name=p + "n1.weight", ffn_norm_name=p + "n2.weight",
                                extra_norms=extra))
    return ModelSpec(architecture=cfg.architecture, hidden_size=H, vocab_size=cfg.vocab_size, layers=tuple(layers),
                     schedule=(ScheduleEntry(0), ScheduleEntry(1)), final_norm=norm, embedding_name="toy.embed.weight",
                     final_norm_name="toy.norm.weight", lm_head_name=None, embedding_scale=1.0, max_position=256,
                     bos_token_id=None, eos_token_id=None)


def plain_sandwich(w, ids):
    x = P.embed(w["toy.embed.weight"], ids, 1.0)
    a = dict(heads=4, kv_heads=2, head_dim=16, rope_theta=1e4, window=24, scale=0.25)
    for i in (0, 1):
        p = f"toy.{i}."
        y = P.attention_layer(P.rmsnorm(x, w[p + "n1.weight"], 1e-5), *(w[p + f"mix.{k}_proj.weight"] for k in "qkvo"), **a)
        x = x + P.rmsnorm(y, w[p + "post1.weight"], 1e-3)
        if i == 0:
            y = P.ffn_layer(P.rmsnorm(x, w[p + "n2.weight"], 1e-5), w[p + "ffn.gate_proj.weight"],
                            w[p + "ffn.up_proj.weight"], w[p + "ffn.down_proj.weight"])
            x = x + P.rmsnorm(y, w[p + "post2.weight"], 1e-3)
    return P.matmul(P.rmsnorm(x, w["toy.norm.weight"], 1e-5), w["toy.embed.weight"])


def test_another_block_arrangement_with_more_norms_and_a_layer_without_feed_forward():
    """A block class registered from here, norms after the mixer and the feed-forward named in the layer
    specification, one layer that has no feed-forward: built, loaded by name and stepped (prompts,
    then tokens one by one) without a change to the framework's files."""
    from inference_engine_rust_b200 import LoadedModel, register_architecture
    from inference_engine_rust_b200.config import registry
    from inference_engine_rust_b200.parts import register_part, unregister_part
    from inference_engine_rust_b200.weights import RandomSource
    register_part("block", "sandwich", SandwichBlock)
    register_architecture("SandwichToyForCausalLM", SandwichConfig, sandwich_spec)
    try:
        raw = {"architectures": ["SandwichToyForCausalLM"], "hidden_size": 64, "vocab_size": 101}
        model = LoadedModel.random(raw, seed=8, dtype="float32", std=0.1)
        names = model.model.expected_tensors()
        assert "toy.0.post2.weight" in names and "toy.1.post1.weight" in names
        assert "toy.1.post2.weight" not in names and "toy.1.n2.weight" not in names and "toy.1.ffn.down_proj.weight" not in names
        src = RandomSource(names, 8, 0.1, dtype=torch.float32)
        w = {n: src.get(n) for n in src.names()}
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(0, 101, (n,), generator=g).tolist() for n in (40, 9)]
        want = [plain_sandwich(w, p) for p in prompts]
        eng = model.session(max_tokens=64 * 4, poison_cache=True).engine
        assert not eng.use_graphs, "a block that does not declare graph_safe keeps graphs off"
        slots = [eng.open_sequence() for _ in prompts]
        tails = [6, 3]
        out = eng.step([(s, p[:len(p) - t]) for s, p, t in zip(slots, prompts, tails)], want="all")
        got, at = [[], []], 0
        for i, (p, t) in enumerate(zip(prompts, tails)):
            got[i].append(out[at:at + len(p) - t].clone())
            at += len(p) - t
        for k in range(max(tails)):
            live = [i for i in range(2) if tails[i] > k]
            out = eng.step([(slots[i], [prompts[i][len(prompts[i]) - tails[i] + k]]) for i in live], want="last")
            for r, i in enumerate(live):
                got[i].append(out[r:r + 1].clone())
        eng.check_device()
        for i in range(2):
            compare(torch.cat(got[i]), want[i], "float32", f"sandwich toy, request {i}")
    finally:
        unregister_part("block", "sandwich")
        registry._ARCHITECTURES.pop("SandwichToyForCausalLM", None)


# ---------------------------------------------------------------------------------------
# another output head, defined here: logits with a soft cap


def _expected_tensors(raw):
    """Names and shapes of a configuration's tensors, from a model built on the device without weights."""
    from inference_engine_rust_b200.config import config_from_dict, spec_of
    from inference_engine_rust_b200.engine.model import Model
    from inference_engine_rust_b200.parts import Runtime
    return Model(spec_of(config_from_dict(raw)), Runtime(torch.float32, "cuda:0")).expected_tensors()


def _soft_cap_head():
    from inference_engine_rust_b200.parts.head import LinearHead

    class SoftCapHead(LinearHead):
        """logits = cap * tanh((hn . W^T) / cap): the linear head, then an element-wise cap (device ops of
        fixed shape, so a captured step stays right)."""
        graph_safe = True

        def __init__(self, spec, hidden_size, vocab_size, rt):
            super().__init__(spec, hidden_size, vocab_size, rt)
            self.cap = float(spec["cap"])

        def forward(self, hn, logits, n_rows, ctx):
            super().forward(hn, logits, n_rows, ctx)
            rows = logits[:n_rows]
            rows.copy_(torch.tanh(rows / self.cap) * self.cap)

    return SoftCapHead


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_another_output_head_is_registered_and_used(dtype):
    """A head kind registered from here and named by the model specification: the engine's logits are the
    plain implementation's with the cap applied, for prompts and for tokens one by one (through captured
    graphs where the run uses them)."""
    import dataclasses
    from helpers import TINY_B
    from inference_engine_rust_b200 import LoadedModel, register_architecture
    from inference_engine_rust_b200.config import registry
    from inference_engine_rust_b200.config.mistral import MistralConfig, build_spec
    from inference_engine_rust_b200.config.specs import PartSpec
    from inference_engine_rust_b200.parts import register_part, unregister_part
    from inference_engine_rust_b200.weights import RandomSource
    from helpers import WEIGHT_STD

    @dataclass(frozen=True)
    class CappedConfig(MistralConfig):                # the same keys; another name, so another specification
        architecture: str = "CappedToyForCausalLM"

    # the plain logits first (the tensor names and shapes are the configuration's own), so that the cap
    # can be put where it binds for some logits and leaves the others nearly alone
    base = dict(TINY_B, architectures=["MistralForCausalLM"])
    src = RandomSource(_expected_tensors(base), 12, WEIGHT_STD, dtype=torch.float32)
    w = {n: src.get(n) for n in src.names()}
    if dtype == "bfloat16":
        w = {n: t.to(torch.bfloat16).float() for n, t in w.items()}
    g = torch.Generator().manual_seed(2)
    ids = torch.randint(0, base["vocab_size"], (29,), generator=g).tolist()
    plain = P.forward(base, w, ids, P.bf16_rounding if dtype == "bfloat16" else P.no_rounding)
    cap = 0.6 * float(plain.abs().max())
    want = torch.tanh(plain / cap) * cap
    assert ((plain - want).abs() > 0.1 * cap).any(), "the cap never binds: the test would not see a head that ignores it"

    register_part("head", "softcap", _soft_cap_head())
    register_architecture("CappedToyForCausalLM", CappedConfig,
                          lambda cfg: dataclasses.replace(build_spec(cfg), head=PartSpec("softcap", {"cap": cap})))
    try:
        raw = dict(TINY_B, architectures=["CappedToyForCausalLM"])
        model = LoadedModel.random(raw, seed=12, dtype=dtype, std=WEIGHT_STD)
        eng = model.session(max_tokens=64 * 2, poison_cache=True).engine
        assert eng.use_graphs
        s = eng.open_sequence()
        got = [eng.step([(s, ids[:20])], want="all").clone()]
        for t in ids[20:]:
            got.append(eng.step([(s, [t])], want="last").clone())
        eng.check_device()
        compare(torch.cat(got), want, dtype, "capped head")
    finally:
        unregister_part("head", "softcap")
        registry._ARCHITECTURES.pop("CappedToyForCausalLM", None)


def test_a_part_that_reads_host_lists_in_a_captured_step_is_refused(toy_registered, monkeypatch):
    """A mixer that declares graph_safe but takes the step's sequences from the host lists would have the
    sequences of the capture frozen into its launches: the capture raises instead of going wrong later."""
    from inference_engine_rust_b200 import LoadedModel
    from inference_engine_rust_b200.parts import register_part

    class Overconfident(RunningMeanMixer):
        graph_safe = True

    register_part("mixer", "running_mean", Overconfident, replace=True)
    try:
        raw = {"architectures": ["ToyForCausalLM"], "hidden_size": 64, "vocab_size": 97, "schedule": [[1, None]]}
        model = LoadedModel.random(raw, seed=4, dtype="float32", std=0.1)
        eng = model.session(max_tokens=64 * 2).engine
        assert eng.use_graphs
        from inference_engine_rust_b200.engine import engine as engine_module
        prompt = [3, 5, 7, 11, 13, 17, 19, 23]
        s = eng.open_sequence()
        eng.step([(s, prompt)], want="last")           # a shape's first prompt is launched one by one
        eng.close_sequence(s)
        s = eng.open_sequence()
        with pytest.raises(RuntimeError, match="graph_safe"):         # its second one is captured
            eng.step([(s, prompt)], want="last")
        eng.close_sequence(s)
        monkeypatch.setattr(engine_module, "PROMPT_GRAPH_MAX_TOKENS", 4)
        s = eng.open_sequence()
        eng.step([(s, prompt)], want="last")           # too long for a captured prompt now: host lists are real
        with pytest.raises(RuntimeError, match="graph_safe"):
            eng.step([(s, [2])], want="last")
    finally:
        register_part("mixer", "running_mean", RunningMeanMixer, replace=True)


# ---------------------------------------------------------------------------------------
# step inputs, defined here: a bias on the embedded rows, and a per-layer input looked up from the
# token ids once per step and read by a later layer's mixer


class EmbedBias:
    """x += bias: changes the embedded rows."""

    def __init__(self, spec, hidden, vocab, rt):
        self.hidden, self.bias = hidden, None

    def tensor_specs(self):
        from inference_engine_rust_b200.weights import TensorSpec
        return {"bias": TensorSpec((self.hidden,))}

    def load(self, tensors):
        self.bias = tensors["bias"].float()

    def prepare(self, tokens, x, ctx):
        x[:ctx.n_tokens] += self.bias


class PerLayerTable:
    """Publishes table[token] ([tokens, width]) as ctx.shared["per_layer"]."""

    def __init__(self, spec, hidden, vocab, rt):
        self.vocab, self.width, self.table = vocab, int(spec["width"]), None

    def tensor_specs(self):
        from inference_engine_rust_b200.weights import TensorSpec
        return {"table": TensorSpec((self.vocab, self.width))}

    def load(self, tensors):
        self.table = tensors["table"].float()

    def prepare(self, tokens, x, ctx):
        ctx.shared["per_layer"] = self.table[tokens[:ctx.n_tokens].long().clamp(min=0)]


class PerLayerMixer:
    """residual += W . (this layer's columns of the per-layer input); it ignores the normed rows."""

    def __init__(self, part_spec, rt):
        self.rt, self.hidden = rt, int(part_spec["hidden_size"])
        self.lo, self.hi = part_spec["columns"]
        self.w = None

    def tensor_specs(self):
        from inference_engine_rust_b200.weights import TensorSpec
        return {"w": TensorSpec((self.hidden, self.hi - self.lo))}

    def load(self, tensors):
        self.w = tensors["w"].float()

    def cache_request(self):
        return None

    def forward(self, xn, residual, ctx, cache_view, writes_cache):
        residual[:ctx.n_tokens] += ctx.shared["per_layer"][:, self.lo:self.hi] @ self.w.t()


@dataclass(frozen=True)
class InputsToyConfig:
    hidden_size: int
    vocab_size: int
    architecture: str = "InputsToyForCausalLM"

    @classmethod
    def from_dict(cls, raw):
        return cls(raw["hidden_size"], raw["vocab_size"])


def inputs_toy_spec(cfg):
    from inference_engine_rust_b200.config.specs import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    H = cfg.hidden_size
    norm = PartSpec("rmsnorm", {"eps": 1e-5})
    attn = PartSpec("attention", {"hidden_size": H, "heads": 4, "kv_heads": 4, "head_dim": 16, "window": None,
                                  "scale": 0.25, "position": PartSpec("rope", {"theta": 1e4, "rotary_dim": 16, "pairing": "half"})})
    ffn = PartSpec("swiglu", {"hidden_size": H, "intermediate_size": 80})
    mixers = (attn, PartSpec("per_layer", {"hidden_size": H, "columns": (4, 12)}))
    layers = tuple(LayerSpec(block=PartSpec("prenorm", {}), norm=norm, mixer=m, ffn=ffn, mixer_prefix=f"toy.{i}.mix.",
                             ffn_prefix=f"toy.{i}.ffn.", mixer_norm_name=f"toy.{i}.n1.weight", ffn_norm_name=f"toy.{i}.n2.weight")
                   for i, m in enumerate(mixers))
    return ModelSpec(architecture=cfg.architecture, hidden_size=H, vocab_size=cfg.vocab_size, layers=layers,
                     schedule=(ScheduleEntry(0), ScheduleEntry(1)), final_norm=norm, embedding_name="toy.embed.weight",
                     final_norm_name="toy.norm.weight", lm_head_name=None, embedding_scale=1.0, max_position=256,
                     bos_token_id=None, eos_token_id=None,
                     inputs=((PartSpec("embed_bias", {}), "toy.in0."), (PartSpec("per_layer_table", {"width": 12}), "toy.in1.")))


def plain_inputs_toy(w, ids):
    x = P.embed(w["toy.embed.weight"], ids, 1.0) + w["toy.in0.bias"]
    per_layer = w["toy.in1.table"][torch.tensor(ids)]
    a = dict(heads=4, kv_heads=4, head_dim=16, rope_theta=1e4, window=None, scale=0.25)
    x = x + P.attention_layer(P.rmsnorm(x, w["toy.0.n1.weight"], 1e-5), *(w[f"toy.0.mix.{k}_proj.weight"] for k in "qkvo"), **a)
    x = x + P.ffn_layer(P.rmsnorm(x, w["toy.0.n2.weight"], 1e-5), *(w[f"toy.0.ffn.{k}_proj.weight"] for k in ("gate", "up", "down")))
    x = x + per_layer[:, 4:12] @ w["toy.1.mix.w"].t()
    x = x + P.ffn_layer(P.rmsnorm(x, w["toy.1.n2.weight"], 1e-5), *(w[f"toy.1.ffn.{k}_proj.weight"] for k in ("gate", "up", "down")))
    return P.matmul(P.rmsnorm(x, w["toy.norm.weight"], 1e-5), w["toy.embed.weight"])


def test_step_inputs_change_the_embedded_rows_and_feed_a_later_layer():
    """Two step inputs registered from here and named by the model specification: one changes the embedded
    rows, one publishes a per-layer input that the second layer's mixer (also defined here, without a
    cache) reads.  Prompts in a batch, then tokens one by one, against the plain statement."""
    from inference_engine_rust_b200 import LoadedModel, register_architecture
    from inference_engine_rust_b200.config import registry
    from inference_engine_rust_b200.parts import register_part, unregister_part
    from inference_engine_rust_b200.weights import RandomSource
    register_part("input", "embed_bias", EmbedBias)
    register_part("input", "per_layer_table", PerLayerTable)
    register_part("mixer", "per_layer", PerLayerMixer)
    register_architecture("InputsToyForCausalLM", InputsToyConfig, inputs_toy_spec)
    try:
        raw = {"architectures": ["InputsToyForCausalLM"], "hidden_size": 64, "vocab_size": 89}
        model = LoadedModel.random(raw, seed=21, dtype="float32", std=0.1)
        names = model.model.expected_tensors()
        assert {"toy.in0.bias", "toy.in1.table", "toy.1.mix.w"} <= set(names)
        src = RandomSource(names, 21, 0.1, dtype=torch.float32)
        w = {n: src.get(n) for n in src.names()}
        g = torch.Generator().manual_seed(5)
        prompts = [torch.randint(0, 89, (n,), generator=g).tolist() for n in (33, 12)]
        want = [plain_inputs_toy(w, p) for p in prompts]
        eng = model.session(max_tokens=64 * 2, poison_cache=True).engine
        assert len(eng.cache.kv_groups) == 1 and sum(len(g.layers) for g in eng.cache.kv_groups) == 1
        slots = [eng.open_sequence() for _ in prompts]
        tails = [5, 2]
        out = eng.step([(s, p[:len(p) - t]) for s, p, t in zip(slots, prompts, tails)], want="all")
        got, at = [[], []], 0
        for i, (p, t) in enumerate(zip(prompts, tails)):
            got[i].append(out[at:at + len(p) - t].clone())
            at += len(p) - t
        for k in range(max(tails)):
            live = [i for i in range(2) if tails[i] > k]
            out = eng.step([(slots[i], [prompts[i][len(prompts[i]) - tails[i] + k]]) for i in live], want="last")
            for r, i in enumerate(live):
                got[i].append(out[r:r + 1].clone())
        eng.check_device()
        for i in range(2):
            compare(torch.cat(got[i]), want[i], "float32", f"step inputs toy, request {i}")
    finally:
        unregister_part("input", "embed_bias")
        unregister_part("input", "per_layer_table")
        unregister_part("mixer", "per_layer")
        registry._ARCHITECTURES.pop("InputsToyForCausalLM", None)
