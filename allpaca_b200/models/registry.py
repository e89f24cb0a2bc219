"""One registry from an architecture's name to how its model is built.

An entry gives the typed configuration class (built from config.json) and a function
from that configuration to a :class:`~allpaca_b200.parts.ModelSpec`.  Both the
``architectures`` entry of config.json and its ``model_type`` are looked up.

The reference has no such table: it matches architecture strings in helpers
(crates/allpaca-gguf/src/parser.rs:885-916, crates/allpaca-core/src/model.rs:3218-3232)
and its safetensors loader accepts any dense SiLU config (model.rs:7908-7919).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping

from ..config.model_config import ConfigError, read_config_json
from ..parts import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type
    spec_builder: Callable[[Any], ModelSpec]


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(names, config_class: type, spec_builder: Callable[[Any], ModelSpec]) -> None:
    for n in ([names] if isinstance(names, str) else names):
        _ARCHITECTURES[n] = Architecture(n, config_class, spec_builder)


def known_architectures():
    return sorted(_ARCHITECTURES)


def resolve(config: Mapping[str, Any]) -> Architecture:
    """The architecture a raw config.json dictionary names."""
    names = list(config.get("architectures") or [])
    if config.get("model_type"):
        names.append(config["model_type"])
    for n in names:
        if n in _ARCHITECTURES:
            return _ARCHITECTURES[n]
    raise ConfigError(
        f"no model is registered for architectures {config.get('architectures')!r} / "
        f"model_type {config.get('model_type')!r} (known: {', '.join(known_architectures())})")


def load_config(path: str):
    """(architecture, typed config) of a model folder or config.json file."""
    raw = read_config_json(path)
    arch = resolve(raw)
    return arch, arch.config_class.from_dict(raw)
