"""The one registry from an architecture's name (``config.json: architectures[0]``) to its model.

An entry holds two callables: ``parse`` turns the raw config.json dictionary into the
architecture's typed configuration, and ``to_spec`` turns that into the architecture-neutral
``ModelSpec`` that the rest of the framework builds from.  Nothing else in the framework names
an architecture.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping

from .specs import ModelSpec


class ConfigError(ValueError):
    """A config.json that is missing a key, has a wrong type, or asks for something unsupported."""


@dataclass(frozen=True)
class Architecture:
    name: str
    parse: Callable[[Mapping[str, Any]], Any]          # raw dict -> typed config (validated)
    to_spec: Callable[[Any], ModelSpec]                # typed config -> ModelSpec
    to_dict: Callable[[Any], Dict[str, Any]]           # typed config -> config.json dict


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture) -> Architecture:
    if arch.name in _ARCHITECTURES:
        raise ValueError(f"architecture {arch.name!r} is already registered")
    _ARCHITECTURES[arch.name] = arch
    return arch


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def get_architecture(name: str) -> Architecture:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        known = ", ".join(sorted(_ARCHITECTURES)) or "(none)"
        raise ConfigError(f"unknown architecture {name!r}; registered: {known}") from None


def registered_architectures():
    return sorted(_ARCHITECTURES)


def architecture_of(raw: Mapping[str, Any]) -> Architecture:
    archs = raw.get("architectures")
    if not isinstance(archs, (list, tuple)) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json needs a non-empty 'architectures' list of strings")
    return get_architecture(archs[0])


def parse_config(raw: Mapping[str, Any]):
    """raw config.json dict -> (Architecture, typed config)."""
    arch = architecture_of(raw)
    return arch, arch.parse(raw)


def load_config(model_dir: str):
    """Reads ``<model_dir>/config.json`` -> (Architecture, typed config)."""
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"cannot open {path}")
    with open(path, "r", encoding="utf-8") as f:
        try:
            raw = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path} is not valid JSON: {e}") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return parse_config(raw)
