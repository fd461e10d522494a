"""Typed configuration of the Mistral / Llama-style dense decoder, read from the keys
of its own config.json, and its `ModelSpec` builder.

Field by field this mirrors what the reference reads from GGUF metadata
(src/model_config.rs:143-306): block count, embedding length, head counts, feed-forward
length, vocabulary, rope theta, rms epsilon, context length, BOS/EOS ids
(src/model_config.rs:35-49).  Differences, on purpose: `head_dim` is a key of its own
(the reference derives hidden/heads, src/model_config.rs:191-197), and `sliding_window`
is honoured (the reference gives this family full causal attention,
src/model_config.rs:505-508, but implements the window mask, src/layers/attention.rs:365-368,
609-613).
"""
from __future__ import annotations

import math
from dataclasses import asdict, dataclass
from typing import Any, Dict, Mapping, Optional

from .registry import ConfigError, register_architecture
from .specs import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE = "MistralForCausalLM"


def _need(raw: Mapping[str, Any], key: str, typ, *, positive: bool = True):
    if key not in raw or raw[key] is None:
        raise ConfigError(f"config.json: required key {key!r} is missing")
    v = raw[key]
    if typ is int:
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError(f"config.json: {key!r} must be an integer, got {v!r}")
    elif typ is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json: {key!r} must be a number, got {v!r}")
        v = float(v)
        if not math.isfinite(v):
            raise ConfigError(f"config.json: {key!r} must be finite, got {v!r}")
    if positive and not v > 0:
        raise ConfigError(f"config.json: {key!r} must be positive, got {v!r}")
    return v


@dataclass(frozen=True)
class MistralConfig:
    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rope_theta: float
    rms_norm_eps: float
    sliding_window: Optional[int]
    max_position_embeddings: int
    tie_word_embeddings: bool
    bos_token_id: Optional[int]
    eos_token_id: Optional[int]
    hidden_act: str = "silu"
    architecture: str = ARCHITECTURE

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "MistralConfig":
        heads = _need(raw, "num_attention_heads", int)
        hidden = _need(raw, "hidden_size", int)
        kv = raw.get("num_key_value_heads")
        if kv is None:
            kv = heads                       # reference default: src/model_config.rs:153-155
        head_dim = raw.get("head_dim")
        if head_dim is None:
            if hidden % heads != 0:          # src/model_config.rs:191-197
                raise ConfigError(
                    f"config.json: hidden_size {hidden} is not divisible by num_attention_heads "
                    f"{heads} and no 'head_dim' is given")
            head_dim = hidden // heads
        window = raw.get("sliding_window")
        act = raw.get("hidden_act", "silu")
        for flag in ("attention_bias", "mlp_bias"):
            if raw.get(flag):
                raise ConfigError(f"config.json: {flag}=true is not supported (this family has no biases)")
        cfg = cls(
            num_hidden_layers=_need(raw, "num_hidden_layers", int),
            hidden_size=hidden,
            num_attention_heads=heads,
            num_key_value_heads=kv,
            head_dim=head_dim,
            intermediate_size=_need(raw, "intermediate_size", int),
            vocab_size=_need(raw, "vocab_size", int),
            rope_theta=float(raw.get("rope_theta", 10000.0)),   # default: src/model_config.rs:160-162
            rms_norm_eps=_need(raw, "rms_norm_eps", float),
            sliding_window=window,
            max_position_embeddings=_need(raw, "max_position_embeddings", int),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            bos_token_id=raw.get("bos_token_id", 1),            # defaults: src/model_config.rs:41-42
            eos_token_id=raw.get("eos_token_id", 2),
            hidden_act=act,
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for key in ("num_key_value_heads", "head_dim"):
            v = getattr(self, key)
            if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
                raise ConfigError(f"config.json: {key!r} must be a positive integer, got {v!r}")
        if self.num_attention_heads % self.num_key_value_heads != 0:   # src/model_config.rs:199-203
            raise ConfigError(
                f"config.json: num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2 != 0:                                      # src/model_config.rs:497-502
            raise ConfigError(f"config.json: head_dim {self.head_dim} must be even for rotary pairs")
        if self.sliding_window is not None:
            w = self.sliding_window
            if isinstance(w, bool) or not isinstance(w, int) or w <= 0:
                raise ConfigError(f"config.json: 'sliding_window' must be null or a positive integer, got {w!r}")
        if self.hidden_act != "silu":                                   # src/layers/ffn.rs:54-56
            raise ConfigError(f"config.json: hidden_act {self.hidden_act!r} is not supported (only 'silu')")
        if not (self.rope_theta > 0 and math.isfinite(self.rope_theta)):
            raise ConfigError(f"config.json: rope_theta must be positive and finite, got {self.rope_theta!r}")
        for key in ("bos_token_id", "eos_token_id"):
            v = getattr(self, key)
            if v is not None and (isinstance(v, bool) or not isinstance(v, int)
                                  or not 0 <= v < self.vocab_size):
                raise ConfigError(f"config.json: {key!r}={v!r} is not a token id below vocab_size")

    def to_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        d.pop("architecture")
        d["architectures"] = [self.architecture]
        d["model_type"] = "mistral"
        return d


def build_spec(cfg: MistralConfig) -> ModelSpec:
    """Every layer: pre-norm block of RMSNorm, rotary GQA attention (optional window),
    SwiGLU (src/layers/block.rs:19-24).  Rotary pairs are (k, k + head_dim/2): the weights
    come in the safetensors row order, where that pairing equals the reference's adjacent
    pairs on its row-permuted GGUF tensors (src/layers/attention.rs:137-172)."""
    norm = PartSpec("rmsnorm", {"eps": cfg.rms_norm_eps})
    position = PartSpec("rope", {
        "theta": cfg.rope_theta,
        "rotary_dim": cfg.head_dim,          # full head: src/model_config.rs:83-89
        "pairing": "half",
    })
    mixer = PartSpec("attention", {
        "hidden_size": cfg.hidden_size,
        "heads": cfg.num_attention_heads,
        "kv_heads": cfg.num_key_value_heads,
        "head_dim": cfg.head_dim,
        "window": cfg.sliding_window,
        "scale": 1.0 / math.sqrt(cfg.head_dim),   # src/layers/attention.rs:357-360
        "position": position,
    })
    ffn = PartSpec("swiglu", {
        "hidden_size": cfg.hidden_size,
        "intermediate_size": cfg.intermediate_size,
    })
    block = PartSpec("prenorm", {})
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        layers.append(LayerSpec(
            block=block, norm=norm, mixer=mixer, ffn=ffn,
            mixer_prefix=p + "self_attn.", ffn_prefix=p + "mlp.",
            mixer_norm_name=p + "input_layernorm.weight",
            ffn_norm_name=p + "post_attention_layernorm.weight"))
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(cfg.num_hidden_layers)),
        final_norm=norm,
        embedding_name="model.embed_tokens.weight",
        final_norm_name="model.norm.weight",
        lm_head_name=None if cfg.tie_word_embeddings else "lm_head.weight",   # src/model_weights/names.rs:300-310
        embedding_scale=1.0,                 # src/model_config.rs:262-265
        max_position=cfg.max_position_embeddings,
        bos_token_id=cfg.bos_token_id,
        eos_token_id=cfg.eos_token_id,
    )


register_architecture(ARCHITECTURE, MistralConfig, build_spec)
