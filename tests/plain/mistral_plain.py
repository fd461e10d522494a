"""Plain, slow implementation of the Mistral / Llama-style decoder, written from the
reference's formulas: whole sequences, no cache, no batching, one function for each part,
CPU float32.  It shares no code with the package under test.

The reference cannot be compiled or imported here (it is a Rust crate and the image has no
Rust toolchain; its own end-to-end tests need a multi-gigabyte GGUF file), so this file
rests on the formulas alone; `tests/test_plain.py` pins each function to the numeric
vectors of the reference's own unit tests.

Every function cites the reference lines it follows (paths inside the reference project).
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional, Sequence

import numpy as np
import torch

Tensor = torch.Tensor
Round = Callable[[Tensor], Tensor]


def no_rounding(t: Tensor) -> Tensor:
    return t


def bf16_rounding(t: Tensor) -> Tensor:
    """Round to bfloat16 and back: where a bfloat16 engine stores an activation."""
    return t.to(torch.bfloat16).to(torch.float32)


# ---------------------------------------------------------------------------------------
# ops


def matmul(x: Tensor, w: Tensor) -> Tensor:
    """out[m, n] = sum_k x[m, k] * w[n, k]; w is [out, in] row-major.
    src/ops/matmul.rs:1-3 (layout), :88-101 (fp32 accumulation)."""
    return x.to(torch.float32) @ w.to(torch.float32).t()


def rmsnorm(x: Tensor, w: Tensor, eps: float) -> Tensor:
    """x * w / sqrt(mean(x^2) + eps) per row.  src/ops/rmsnorm.rs:38-48."""
    x = x.to(torch.float32)
    mean_sq = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    rms = torch.sqrt(mean_sq + torch.tensor(eps, dtype=torch.float32))
    return x * w.to(torch.float32) / rms


def softmax(x: Tensor) -> Tensor:
    """exp(x - max) / sum exp(x - max) over the last axis.  src/ops/softmax.rs:11-25."""
    m = x.max(dim=-1, keepdim=True).values
    e = torch.exp(x - m)
    return e / e.sum(dim=-1, keepdim=True)


def sigmoid(x: Tensor) -> Tensor:
    """Branch-stable sigmoid.  src/ops/swiglu.rs:3-20."""
    pos = 1.0 / (1.0 + torch.exp(-x.clamp(min=0)))
    z = torch.exp(x.clamp(max=0))
    neg = z / (1.0 + z)
    return torch.where(x >= 0, pos, neg)


def swiglu(gate: Tensor, up: Tensor) -> Tensor:
    """gate * sigmoid(gate) * up.  src/ops/swiglu.rs:24-36."""
    return gate * sigmoid(gate) * up


def rope_angles(pos: int, base: float, rotary_dim: int,
                freq_factors: Optional[Sequence[float]] = None) -> Tensor:
    """Angles of the rotary pairs at `pos`: theta starts at pos and is multiplied by
    base^(-2/rotary_dim) per pair, all in float32.  src/ops/rope.rs:40-57."""
    n_pairs = rotary_dim // 2
    theta_scale = np.float32(np.float32(base) ** np.float32(-2.0 / np.float32(rotary_dim))) if rotary_dim else np.float32(1)
    theta = np.float32(pos)
    out = np.zeros(n_pairs, dtype=np.float32)
    for k in range(n_pairs):
        ff = np.float32(1.0)
        if freq_factors is not None and freq_factors[k] != 0:
            ff = np.float32(freq_factors[k])
        out[k] = theta / ff
        theta = np.float32(theta * theta_scale)
    return torch.from_numpy(out)


def rope(vec: Tensor, base: float, pos: int, head_dim: int, rotary_dim: int,
         pairing: str = "interleaved", freq_factors=None) -> Tensor:
    """Rotate one head at position `pos`.  The reference rotates adjacent pairs (2k, 2k+1)
    (src/ops/rope.rs:51-56); on weights in safetensors row order the same rotation pairs
    (k, k + rotary_dim/2) ("half"; background src/layers/attention.rs:137-172).
    Dimensions from rotary_dim on pass through."""
    assert rotary_dim <= head_dim and rotary_dim % 2 == 0
    ang = rope_angles(pos, base, rotary_dim, freq_factors)
    cos, sin = torch.cos(ang), torch.sin(ang)
    out = vec.clone().to(torch.float32)
    half = rotary_dim // 2
    if pairing == "interleaved":
        i0 = torch.arange(half) * 2
        i1 = i0 + 1
    elif pairing == "half":
        i0 = torch.arange(half)
        i1 = i0 + half
    else:
        raise ValueError(pairing)
    a, b = vec[i0].to(torch.float32), vec[i1].to(torch.float32)
    out[i0] = a * cos - b * sin
    out[i1] = a * sin + b * cos
    return out


def rope_sequence(x: Tensor, base: float, head_dim: int, rotary_dim: int, pairing: str,
                  first_pos: int = 0, positions: Optional[Sequence[int]] = None) -> Tensor:
    """`rope` on every head of every row of x [T, heads, head_dim]; row t is at position
    first_pos + t (prefill: the row index, src/layers/attention.rs:314-343).  `positions`
    overrides that (only the tests that plant a fault use it)."""
    out = x.clone().to(torch.float32)
    half = rotary_dim // 2
    if pairing == "interleaved":
        i0 = torch.arange(half) * 2
        i1 = i0 + 1
    else:
        i0 = torch.arange(half)
        i1 = i0 + half
    for t in range(x.shape[0]):
        ang = rope_angles(first_pos + t if positions is None else positions[t], base, rotary_dim)
        cos, sin = torch.cos(ang), torch.sin(ang)
        a, b = x[t][:, i0].to(torch.float32), x[t][:, i1].to(torch.float32)
        out[t][:, i0] = a * cos - b * sin
        out[t][:, i1] = a * sin + b * cos
    return out


def embed(table: Tensor, ids: Sequence[int], scale: float = 1.0) -> Tensor:
    """x[t, :] = table[ids[t], :] * scale; an id outside the table is an error.
    src/layers/embeddings.rs:15-17,119-139; src/engine/embed.rs:140-149."""
    vocab = table.shape[0]
    for i in ids:
        if not 0 <= i < vocab:
            raise ValueError(f"token id {i} out of range")
    return table[torch.tensor(list(ids), dtype=torch.long)].to(torch.float32) * scale


# ---------------------------------------------------------------------------------------
# layers


def attention_layer(xn: Tensor, wq: Tensor, wk: Tensor, wv: Tensor, wo: Tensor, *, heads: int,
                    kv_heads: int, head_dim: int, rope_theta: float, window: Optional[int],
                    pairing: str = "half", rotary_dim: Optional[int] = None,
                    scale: Optional[float] = None, rnd: Round = no_rounding,
                    return_parts: bool = False, kv_head_of: Optional[Callable[[int], int]] = None,
                    positions: Optional[Sequence[int]] = None):
    """Attention of one whole sequence starting at position 0.
    Projections src/layers/attention.rs:245-254; rotation of every Q and K head at its row
    index :314-343; scores over j in [j_min, pos] with j_min = pos - (window - 1), scaled by
    1/sqrt(head_dim), softmax, weighted values :357-415 (grouped heads: kv_head =
    head / (heads / kv_heads), :372); output projection :417-421.
    `kv_head_of` and `positions` replace the head grouping and the row positions; they exist
    for the tests that plant a fault and check that the tolerances catch it."""
    T = xn.shape[0]
    rotary_dim = head_dim if rotary_dim is None else rotary_dim
    scale = 1.0 / math.sqrt(head_dim) if scale is None else scale
    q = rnd(matmul(xn, wq)).view(T, heads, head_dim)
    k = rnd(matmul(xn, wk)).view(T, kv_heads, head_dim)
    v = rnd(matmul(xn, wv)).view(T, kv_heads, head_dim)
    q_r = rope_sequence(q, rope_theta, head_dim, rotary_dim, pairing, positions=positions)
    k_r = rope_sequence(k, rope_theta, head_dim, rotary_dim, pairing, positions=positions)
    q_r, k_r = rnd(q_r), rnd(k_r)
    group = heads // kv_heads
    out = torch.zeros(T, heads, head_dim, dtype=torch.float32)
    rows = torch.arange(T).view(T, 1)
    cols = torch.arange(T).view(1, T)
    visible = cols <= rows
    if window is not None:
        visible = visible & (cols >= rows - (window - 1))
    for h in range(heads):
        kvh = h // group if kv_head_of is None else kv_head_of(h)
        scores = (q_r[:, h] @ k_r[:, kvh].t()) * scale
        scores = scores.masked_fill(~visible, float("-inf"))
        p = softmax(scores)
        out[:, h] = p @ v[:, kvh]
    attn = rnd(out.reshape(T, heads * head_dim))
    y = matmul(attn, wo)
    if return_parts:
        return y, {"q": q_r, "k": k_r, "v": v, "attn": attn}
    return y


def ffn_layer(xn: Tensor, w_gate: Tensor, w_up: Tensor, w_down: Tensor, rnd: Round = no_rounding) -> Tensor:
    """down(swiglu(gate(x), up(x))).  src/layers/ffn.rs:35-63."""
    g = rnd(matmul(xn, w_gate))
    u = rnd(matmul(xn, w_up))
    return matmul(rnd(swiglu(g, u)), w_down)


def block(x: Tensor, cfg: dict, w: Dict[str, Tensor], layer: int, rnd: Round = no_rounding,
          **attention_options) -> Tensor:
    """x += attention(norm(x)); x += ffn(norm(x)).  src/layers/block.rs:19-24;
    residual on the un-normed input src/layers/attention.rs:757-759, src/layers/ffn.rs:113-116."""
    p = f"model.layers.{layer}."
    eps = cfg["rms_norm_eps"]
    xn = rnd(rmsnorm(x, w[p + "input_layernorm.weight"], eps))
    x = x + attention_layer(
        xn, w[p + "self_attn.q_proj.weight"], w[p + "self_attn.k_proj.weight"],
        w[p + "self_attn.v_proj.weight"], w[p + "self_attn.o_proj.weight"],
        heads=cfg["num_attention_heads"], kv_heads=cfg["num_key_value_heads"],
        head_dim=cfg["head_dim"], rope_theta=cfg["rope_theta"], window=cfg.get("sliding_window"),
        rnd=rnd, **attention_options)
    xn = rnd(rmsnorm(x, w[p + "post_attention_layernorm.weight"], eps))
    x = x + ffn_layer(xn, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                      w[p + "mlp.down_proj.weight"], rnd)
    return x


def forward(cfg: dict, w: Dict[str, Tensor], ids: Sequence[int], rnd: Round = no_rounding,
            **attention_options) -> Tensor:
    """Logits [len(ids), vocab] of one whole sequence.  Embedding src/engine/embed.rs:104-138;
    layer loop src/engine/runtime.rs:27-31; final norm and output head :89-107 (there for the
    last row only; here for every row); tied output src/model_weights/names.rs:300-310."""
    if len(ids) == 0:
        raise ValueError("empty prompt")                      # src/engine/embed.rs:109-111
    x = embed(w["model.embed_tokens.weight"], ids, 1.0)
    for layer in range(cfg["num_hidden_layers"]):
        x = block(x, cfg, w, layer, rnd, **attention_options)
    hn = rnd(rmsnorm(x, w["model.norm.weight"], cfg["rms_norm_eps"]))
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else w["lm_head.weight"]
    return matmul(hn, head)


# ---------------------------------------------------------------------------------------
# sampling


def sample_greedy(logits: Sequence[float]) -> int:
    """First index of the largest logit; empty or non-finite input is an error.
    src/engine/sampling.rs:25-49."""
    if len(logits) == 0:
        raise ValueError("empty logits")
    best, best_v = 0, None
    for i, v in enumerate(logits):
        v = float(v)
        if not math.isfinite(v):
            raise ValueError("non-finite logit")
        if best_v is None or v > best_v:
            best, best_v = i, v
    return best


def temperature_cdf(logits: Tensor, temperature: float) -> Tensor:
    """Running sums of softmax(logits / T) in vocabulary order (float64 for a sharp oracle).
    src/engine/sampling.rs:66-72."""
    if not (math.isfinite(temperature) and temperature > 0):
        raise ValueError(f"temperature must be positive, got {temperature}")     # :62-64
    scaled = logits.to(torch.float64) / temperature
    p = torch.exp(scaled - scaled.max())
    p = p / p.sum()
    return torch.cumsum(p, dim=0)


def sample_temperature(logits: Tensor, temperature: float, r: float) -> int:
    """First i with r < cum_i, else the last index.  src/engine/sampling.rs:70-78."""
    if logits.numel() == 0:
        raise ValueError("empty logits")
    cdf = temperature_cdf(logits, temperature)
    hits = torch.nonzero(cdf > r)
    return int(hits[0]) if hits.numel() else logits.numel() - 1


def philox4x32_10(counter: Sequence[int], key: Sequence[int]) -> List[int]:
    """Philox4x32 with 10 rounds (Salmon, Moraes, Dror, Shaw 2011).  Not from the reference,
    which takes the caller's generator (src/engine/sampling.rs:54-58): the package under
    test states that its uniform draw is the top 24 bits of the first output word for
    counter (request, step, 0, 0) and key (seed low, seed high); this is an independent
    statement of that generator."""
    M0, M1, W0, W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
    c = [int(x) & 0xFFFFFFFF for x in counter]
    k = [int(x) & 0xFFFFFFFF for x in key]
    for _ in range(10):
        p0, p1 = M0 * c[0], M1 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k[0]) & 0xFFFFFFFF, p1 & 0xFFFFFFFF,
             ((p0 >> 32) ^ c[3] ^ k[1]) & 0xFFFFFFFF, p0 & 0xFFFFFFFF]
        k = [(k[0] + W0) & 0xFFFFFFFF, (k[1] + W1) & 0xFFFFFFFF]
    return c


def uniform_draw(seed: int, request: int, step: int) -> float:
    out = philox4x32_10([request, step, 0, 0], [seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF])
    return (out[0] >> 8) / 16777216.0


def generate_greedy(cfg: dict, w: Dict[str, Tensor], prompt: Sequence[int], new_tokens: int,
                    stop_ids=()) -> List[int]:
    """The reference's loop with the whole sequence run again for every token
    (teacher forcing): src/main.rs:102-116, tests/gemma_decode_self_consistency.rs:219-320."""
    ids = list(prompt)
    out: List[int] = []
    for _ in range(new_tokens):
        nxt = sample_greedy(forward(cfg, w, ids)[-1].tolist())
        if nxt in stop_ids:
            break
        out.append(nxt)
        ids.append(nxt)
    return out
