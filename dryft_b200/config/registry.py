"""One registry from an architecture's name (``config.json["architectures"][0]``) to what
builds it.  The reference never reads ``architectures``; it serves one pinned checkpoint
(``engine/dryft_qwen3/config.py:55-70``).  Here the name picks the typed configuration,
and the configuration yields the ``ModelSpec`` every other component works from.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping

from .spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    """``config_from_dict`` parses config.json into a typed configuration object that has
    ``model_spec() -> ModelSpec`` and ``to_dict() -> dict``."""

    name: str
    config_from_dict: Callable[[Mapping[str, Any]], Any]


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_from_dict: Callable[[Mapping[str, Any]], Any]) -> None:
    _ARCHITECTURES[name] = Architecture(name, config_from_dict)


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def known_architectures() -> list:
    return sorted(_ARCHITECTURES)


def architecture_of(raw: Mapping[str, Any]) -> Architecture:
    archs = raw.get("architectures")
    if not archs or not isinstance(archs, (list, tuple)):
        raise KeyError("config.json: 'architectures' is missing or empty; known: " + ", ".join(known_architectures()))
    name = archs[0]
    if name not in _ARCHITECTURES:
        raise KeyError(f"config.json: unknown architecture {name!r}; known: " + ", ".join(known_architectures()))
    return _ARCHITECTURES[name]


def config_from_dict(raw: Mapping[str, Any]) -> Any:
    return architecture_of(raw).config_from_dict(raw)


def load_config(model_dir: str) -> Any:
    """Typed configuration of the model folder, its class chosen by ``architectures``."""
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"{path}: not found (a model folder holds config.json and model.safetensors)")
    with open(path, "r", encoding="utf-8") as f:
        raw = json.load(f)
    return config_from_dict(raw)


def load_model_spec(model_dir: str) -> ModelSpec:
    return load_config(model_dir).model_spec()
