"""Weights: read from safetensors by tensor name, or made at random from a seed."""

from .checkpoint import Checkpoint, WeightsError, shard_files
from .expected import expected_tensors
from .random_init import random_state_dict, write_random_model
from .source import CheckpointSource, RandomSource, WeightSource, random_tensor, resolve_dtype

__all__ = [
    "Checkpoint", "CheckpointSource", "RandomSource", "WeightSource", "WeightsError", "expected_tensors",
    "random_state_dict", "random_tensor", "resolve_dtype", "shard_files", "write_random_model",
]
