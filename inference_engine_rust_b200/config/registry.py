"""One registry from an architecture's name (config.json `architectures[0]`) to its
typed configuration class and its spec builder.

The reference picks a family by string match and then branches on it at each call site
(src/model_config.rs:461-482, src/layers/attention.rs:703-710).  Here the branch happens
once: the registered builder emits a `ModelSpec`, and nothing below it knows the name.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping, Type

from .specs import ModelSpec


class ConfigError(ValueError):
    """A configuration that cannot be built (missing key, bad value, unknown name)."""


@dataclass(frozen=True)
class ArchitectureEntry:
    name: str
    config_cls: Type[Any]                      # has from_dict(mapping) and to_dict()
    build_spec: Callable[[Any], ModelSpec]     # typed config -> ModelSpec


_ARCHITECTURES: Dict[str, ArchitectureEntry] = {}


def register_architecture(name: str, config_cls: Type[Any],
                          build_spec: Callable[[Any], ModelSpec]) -> None:
    if name in _ARCHITECTURES:
        raise ConfigError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = ArchitectureEntry(name, config_cls, build_spec)


def known_architectures() -> list:
    return sorted(_ARCHITECTURES)


def architecture(name: str) -> ArchitectureEntry:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"unknown architecture {name!r}; registered: {known_architectures()}") from None


def architecture_name_of(raw: Mapping[str, Any]) -> str:
    archs = raw.get("architectures")
    if not isinstance(archs, (list, tuple)) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json: key 'architectures' must be a non-empty list of names")
    return archs[0]


def config_from_dict(raw: Mapping[str, Any]):
    """Typed configuration for whatever architecture `raw` names."""
    entry = architecture(architecture_name_of(raw))
    return entry.config_cls.from_dict(raw)


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            raw = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"{path}: not found") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return raw


def load_config(model_dir: str):
    return config_from_dict(read_config_json(model_dir))


def spec_of(config) -> ModelSpec:
    """The `ModelSpec` of a typed configuration (looked up by its architecture name)."""
    entry = architecture(config.architecture)
    spec = entry.build_spec(config)
    spec.validate()
    return spec
