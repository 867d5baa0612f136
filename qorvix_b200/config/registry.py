"""One registry from an architecture's name to its configuration class and model builder.

The reference keeps an allow-list of architecture strings (runtime/src/model_config.cpp:20-38)
and a plugin registry keyed by architecture that refuses duplicates
(core/src/plugin_registry.cpp:47-51).  Here one table does both: `architectures[0]` of
config.json selects an entry; the entry turns the raw dict into a typed configuration and
the configuration into a ModelSpec (the list of layers and their parts).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict

from .model_config import ConfigError, ModelConfig, read_config_json


@dataclass(frozen=True)
class ArchitectureEntry:
    name: str
    config_from_dict: Callable[[dict], ModelConfig]
    build_spec: Callable[[ModelConfig], "object"]          # -> parts.spec.ModelSpec
    random_tensors: Callable[..., "object"] = None          # (config, seed, device) -> iterator of (name, tensor)


_ARCHITECTURES: Dict[str, ArchitectureEntry] = {}


def register_architecture(name: str, config_from_dict, build_spec, random_tensors=None, *, replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture '{name}' is already registered")
    _ARCHITECTURES[name] = ArchitectureEntry(name, config_from_dict, build_spec, random_tensors)


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def registered_architectures() -> list:
    return sorted(_ARCHITECTURES)


def lookup_architecture(name: str) -> ArchitectureEntry:
    if name not in _ARCHITECTURES:
        raise ConfigError(f"architecture '{name}' is not registered (known: {', '.join(registered_architectures()) or 'none'})")
    return _ARCHITECTURES[name]


def architecture_of(raw: dict) -> str:
    archs = raw.get("architectures")
    if not archs:
        raise ConfigError("config.json: required key 'architectures' is missing")
    return str(archs[0])


def load_config(model_dir) -> ModelConfig:
    """config.json of a model folder -> the typed configuration of its architecture."""
    raw = read_config_json(model_dir)
    return lookup_architecture(architecture_of(raw)).config_from_dict(raw)
