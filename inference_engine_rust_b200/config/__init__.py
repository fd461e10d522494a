"""Typed configurations, the architecture registry and the architecture-neutral specs."""
from .registry import (ConfigError, architecture, architecture_name_of, config_from_dict,
                       known_architectures, load_config, read_config_json,
                       register_architecture, spec_of)
from .specs import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .mistral import MistralConfig  # registers "MistralForCausalLM"
from .presets import PRESETS, preset

__all__ = [
    "ConfigError", "architecture", "architecture_name_of", "config_from_dict",
    "known_architectures", "load_config", "read_config_json", "register_architecture",
    "spec_of", "LayerSpec", "ModelSpec", "PartSpec", "ScheduleEntry", "MistralConfig", "PRESETS", "preset",
]
