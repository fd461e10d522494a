"""Architecture-neutral description of a model: what every layer is made of and in
which order layers run.

A `ModelSpec` is plain data.  An architecture's builder (see `registry.py`) turns its
typed configuration into one; the engine then assembles parts from it without knowing
which architecture it came from.  The reference keeps the same information in
per-layer vectors (`LayerDims`, `LayerAttentionSpec`: src/model_config.rs:74-100,115,127).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Sequence, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: the registered `kind` and that kind's own parameters."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    """A layer = block arrangement + norms + mixer + feed-forward, with the tensor-name
    prefixes under which each part finds its weights.

    The usual layer has two norms of one kind (before the mixer, before the feed-forward).  A block
    arrangement that needs more (norms after the mixer or the feed-forward, a norm of another kind)
    names them in `extra_norms`: role -> (spec, weight tensor name); its block class receives them
    built, by role.  `ffn` may be None for a layer that has no feed-forward."""

    block: PartSpec            # arrangement, e.g. kind "prenorm"
    norm: PartSpec             # the norm used before the mixer and before the feed-forward
    mixer: PartSpec            # token mixer, e.g. kind "attention"
    ffn: Optional[PartSpec]    # feed-forward, e.g. kind "swiglu"; None: the layer has none
    mixer_prefix: str          # e.g. "model.layers.3.self_attn."
    ffn_prefix: str            # e.g. "model.layers.3.mlp."
    mixer_norm_name: str       # e.g. "model.layers.3.input_layernorm.weight"
    ffn_norm_name: str         # e.g. "model.layers.3.post_attention_layernorm.weight"
    extra_norms: Mapping[str, Tuple[PartSpec, str]] = field(default_factory=dict)


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a layer.  `layer` indexes `ModelSpec.layers`; a layer may be named
    by several entries (shared weights), and each entry that writes a cache has storage of
    its own.  `reads_cache_of` names an EARLIER entry of the schedule (by its position)
    whose cache this execution reads instead of writing one."""

    layer: int
    reads_cache_of: Optional[int] = None

    @property
    def writes_cache(self) -> bool:
        return self.reads_cache_of is None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    layers: Sequence[LayerSpec]
    schedule: Sequence[ScheduleEntry]
    final_norm: PartSpec
    embedding_name: str
    final_norm_name: str
    lm_head_name: Optional[str]       # None = output tied to the embedding table
    embedding_scale: float
    max_position: int
    bos_token_id: Optional[int]
    eos_token_id: Optional[int]
    head: PartSpec = PartSpec("linear")   # what turns the final norm's rows into logits
    # Parts that run once per step, after the embedding and before the first block: (spec, tensor-name prefix).
    # Each may change the embedded rows and publish tensors for the blocks (a per-layer input, say).
    inputs: Sequence[Tuple[PartSpec, str]] = ()

    def validate(self) -> None:
        n = len(self.layers)
        if n == 0:
            raise ValueError("model has no layers")
        if not self.schedule:
            raise ValueError("layer schedule is empty")
        for pos, e in enumerate(self.schedule):
            if not 0 <= e.layer < n:
                raise ValueError(f"schedule entry {pos} names layer {e.layer}, the model has {n}")
            if e.reads_cache_of is not None:
                src = e.reads_cache_of
                if not 0 <= src < pos:
                    raise ValueError(
                        f"schedule entry {pos} reads the cache of entry {src}, which does not run before it")
                if not self.schedule[src].writes_cache:
                    raise ValueError(
                        f"schedule entry {pos} reads the cache of entry {src}, which writes none")

    def cache_entry(self, pos: int) -> int:
        """Position of the schedule entry whose cache entry `pos` uses."""
        e = self.schedule[pos]
        return pos if e.reads_cache_of is None else e.reads_cache_of
