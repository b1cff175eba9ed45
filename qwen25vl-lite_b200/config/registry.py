"""The one registry from an architecture's name (``config.json["architectures"][0]``) to
its model: a typed configuration class and a spec builder.

The reference has no such table: it stores ``model_type`` and never dispatches on it
(src/qwen25vl_lite/config.py:150,191) and hard-wires one model class
(src/qwen25vl_lite/cli.py:108).  Here every entry point (generation, replay, bench, random
weights) resolves the model through :func:`resolve_architecture`.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict

from .spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    config_from_dict: Callable[[Dict[str, Any]], Any]   # whole config.json -> typed config
    build_spec: Callable[[Any], ModelSpec]              # typed config -> ModelSpec


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_from_dict, build_spec, *, replace: bool = False) -> Architecture:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {name!r} is already registered")
    arch = Architecture(name, config_from_dict, build_spec)
    _ARCHITECTURES[name] = arch
    return arch


def known_architectures():
    return sorted(_ARCHITECTURES)


def resolve_architecture(raw_config: Dict[str, Any]) -> Architecture:
    names = raw_config.get("architectures")
    if not names:
        raise ValueError(
            "config.json has no 'architectures' entry; known architectures: " + ", ".join(known_architectures()))
    name = names[0]
    if name not in _ARCHITECTURES:
        raise ValueError(f"unknown architecture {name!r}; known architectures: " + ", ".join(known_architectures()))
    return _ARCHITECTURES[name]
