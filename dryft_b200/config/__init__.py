"""Typed configurations, the architecture registry and the architecture-neutral model spec."""

from .spec import ExtraPart, LayerSpec, ModelSpec, PartSpec, RunStep
from .qwen3 import ConfigError, Qwen3Config
from .registry import (
    Architecture,
    architecture_of,
    config_from_dict,
    known_architectures,
    load_config,
    load_model_spec,
    register_architecture,
    unregister_architecture,
)
from .presets import PRESETS, preset

register_architecture("Qwen3ForCausalLM", Qwen3Config.from_dict)

__all__ = [
    "ExtraPart",
    "Architecture", "ConfigError", "LayerSpec", "ModelSpec", "PartSpec", "PRESETS", "Qwen3Config", "RunStep",
    "architecture_of", "config_from_dict", "known_architectures", "load_config", "load_model_spec",
    "preset", "register_architecture", "unregister_architecture",
]
