"""The parts a layer is put together from: mixers, feed-forwards, norms, position encodings, block
arrangements, the embedding and the output head.  Importing this package registers the built-in
kinds; ``register_*`` adds others without touching any file here."""

from .base import (
    BLOCKS, EMBEDDINGS, FFNS, HEADS, MIXERS, NORMS, POSITIONS, Registry, Residual, Runtime, StepContext, TensorInfo,
    register_block, register_embedding, register_ffn, register_head, register_mixer, register_norm, register_position,
)
from . import attention, block, embedding, ffn, norm, position  # noqa: F401  (registration)
from .linear import linear

__all__ = [
    "BLOCKS", "EMBEDDINGS", "FFNS", "HEADS", "MIXERS", "NORMS", "POSITIONS", "Registry", "Residual", "Runtime", "StepContext",
    "TensorInfo", "linear", "register_block", "register_embedding", "register_ffn", "register_head", "register_mixer",
    "register_norm", "register_position",
]
