"""Typed configuration of the Qwen3 dense decoder, read from its own ``config.json`` keys.

Parity: ``engine/dryft_qwen3/config.py:73-155`` (``ModelConfig`` / ``load_model_config``).
Differences, on purpose: no pinned checkpoint (any Qwen3 dense size loads), failed
checks are ``ConfigError`` naming the key instead of bare asserts, an untied
``lm_head`` is allowed, and ``use_sliding_window`` selects windowed attention per
layer instead of being refused (``config.py:140``).

No size or constant that ``config.json`` gives appears as a literal below.
"""

from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .spec import LayerSpec, ModelSpec, PartSpec, RunStep


class ConfigError(ValueError):
    """A ``config.json`` that this library cannot serve; the message names the key."""


_REQUIRED = (
    "num_hidden_layers",
    "hidden_size",
    "num_attention_heads",
    "num_key_value_heads",
    "intermediate_size",
    "vocab_size",
    "rms_norm_eps",
    "max_position_embeddings",
)

FULL_ATTENTION = "full_attention"
SLIDING_ATTENTION = "sliding_attention"


def _positive_int(raw: Mapping[str, Any], key: str) -> int:
    v = raw[key]
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {key} must be a positive integer, got {v!r}")
    return v


@dataclass(frozen=True)
class Qwen3Config:
    """Field names are the ``config.json`` keys (``engine/dryft_qwen3/config.py:142-155``)."""

    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    max_position_embeddings: int
    hidden_act: str = "silu"
    layer_types: Tuple[str, ...] = ()
    sliding_window: Optional[int] = None
    architecture: str = "Qwen3ForCausalLM"

    # ------------------------------------------------------------------ derived sizes
    @property
    def q_dim(self) -> int:
        """Width of the query projection; need not equal ``hidden_size`` (``config.py:87-89``)."""
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def group(self) -> int:
        """Query heads per key/value head (``config.py:99-101``)."""
        return self.num_attention_heads // self.num_key_value_heads

    @property
    def attention_scale(self) -> float:
        """``1/sqrt(head_dim)`` (``engine/dryft_qwen3/model.py:65``)."""
        return 1.0 / math.sqrt(self.head_dim)

    def kv_bytes_per_token(self, itemsize: int) -> int:
        """Cache bytes one token holds over all layers (``config.py:103-105``)."""
        return self.num_hidden_layers * 2 * self.kv_dim * itemsize

    def weight_bytes_per_decode_step(self, itemsize: int) -> int:
        """Bytes of weights one decode step has to read: every matrix once, the output
        head once (the embedding rows it gathers are negligible) — ``config.py:107-115``."""
        per_layer = (self.q_dim + 2 * self.kv_dim) * self.hidden_size + self.hidden_size * self.q_dim
        per_layer += 3 * self.intermediate_size * self.hidden_size
        return itemsize * (self.num_hidden_layers * per_layer + self.vocab_size * self.hidden_size)

    def matmul_flops_per_token(self) -> int:
        """Multiply-add flops of the weight matrices for one token, output head excluded."""
        per_layer = (self.q_dim + 2 * self.kv_dim) * self.hidden_size + self.hidden_size * self.q_dim
        per_layer += 3 * self.intermediate_size * self.hidden_size
        return 2 * self.num_hidden_layers * per_layer

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "Qwen3Config":
        missing = [k for k in _REQUIRED if k not in raw]
        theta = raw.get("rope_theta")
        if theta is None and isinstance(raw.get("rope_parameters"), Mapping):
            theta = raw["rope_parameters"].get("rope_theta")
        if theta is None:
            missing.append("rope_theta")
        if missing:
            raise ConfigError("config.json: missing required key(s): " + ", ".join(missing))

        layers = _positive_int(raw, "num_hidden_layers")
        hidden = _positive_int(raw, "hidden_size")
        heads = _positive_int(raw, "num_attention_heads")
        kv_heads = _positive_int(raw, "num_key_value_heads")
        inter = _positive_int(raw, "intermediate_size")
        vocab = _positive_int(raw, "vocab_size")
        max_pos = _positive_int(raw, "max_position_embeddings")
        if heads % kv_heads != 0:
            raise ConfigError(
                f"config.json: num_attention_heads ({heads}) must be a multiple of num_key_value_heads ({kv_heads})"
            )
        # head_dim defaults to hidden_size // num_attention_heads (config.py:142)
        head_dim = raw.get("head_dim") or hidden // heads
        if isinstance(head_dim, bool) or not isinstance(head_dim, int) or head_dim <= 0 or head_dim % 2:
            raise ConfigError(f"config.json: head_dim must be a positive even integer, got {head_dim!r}")
        eps = float(raw["rms_norm_eps"])
        if not eps > 0.0:
            raise ConfigError(f"config.json: rms_norm_eps must be positive, got {raw['rms_norm_eps']!r}")
        theta = float(theta)
        if not theta > 0.0:
            raise ConfigError(f"config.json: rope_theta must be positive, got {theta!r}")
        act = raw.get("hidden_act", "silu")
        if act != "silu":  # config.py:137
            raise ConfigError(f"config.json: hidden_act {act!r} is not supported (only 'silu')")
        if raw.get("attention_bias", False):  # config.py:138
            raise ConfigError("config.json: attention_bias=true is not supported (Qwen3 dense has no biases)")
        scaling = raw.get("rope_scaling")
        if scaling is None and isinstance(raw.get("rope_parameters"), Mapping):
            rtype = raw["rope_parameters"].get("rope_type", "default")
            scaling = None if rtype == "default" else raw["rope_parameters"]
        if scaling is not None:  # config.py:139
            raise ConfigError(f"config.json: rope_scaling {scaling!r} is not supported (only null)")

        # Windowed layers: Qwen3's own keys.  With use_sliding_window the layers from
        # max_window_layers on see only the last sliding_window keys, unless layer_types
        # lists every layer explicitly.
        window = None
        types: Tuple[str, ...]
        if raw.get("use_sliding_window", False):
            window = raw.get("sliding_window")
            if isinstance(window, bool) or not isinstance(window, int) or window <= 0:
                raise ConfigError(f"config.json: use_sliding_window needs a positive sliding_window, got {window!r}")
            if raw.get("layer_types") is not None:
                types = tuple(raw["layer_types"])
            else:
                first = raw.get("max_window_layers", layers)
                if isinstance(first, bool) or not isinstance(first, int) or first < 0:
                    raise ConfigError(f"config.json: max_window_layers must be a non-negative integer, got {first!r}")
                types = tuple(SLIDING_ATTENTION if i >= first else FULL_ATTENTION for i in range(layers))
        else:
            types = tuple(FULL_ATTENTION for _ in range(layers))
        if len(types) != layers:
            raise ConfigError(f"config.json: layer_types has {len(types)} entries for {layers} layers")
        for t in types:
            if t not in (FULL_ATTENTION, SLIDING_ATTENTION):
                raise ConfigError(f"config.json: layer_types entry {t!r} is not supported")
        if all(t == FULL_ATTENTION for t in types):
            window = None

        archs = raw.get("architectures") or ["Qwen3ForCausalLM"]
        return cls(
            num_hidden_layers=layers,
            hidden_size=hidden,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            intermediate_size=inter,
            vocab_size=vocab,
            rms_norm_eps=eps,
            rope_theta=theta,
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),  # config.py:153
            max_position_embeddings=max_pos,
            hidden_act=act,
            layer_types=types,
            sliding_window=window,
            architecture=str(archs[0]),
        )

    @classmethod
    def from_model_dir(cls, model_dir: str) -> "Qwen3Config":
        with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> dict:
        """The ``config.json`` this configuration is read back from."""
        d = {
            "architectures": [self.architecture],
            "model_type": "qwen3",
            "num_hidden_layers": self.num_hidden_layers,
            "hidden_size": self.hidden_size,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": None,
            "tie_word_embeddings": self.tie_word_embeddings,
            "max_position_embeddings": self.max_position_embeddings,
            "hidden_act": self.hidden_act,
            "attention_bias": False,
            "use_sliding_window": self.sliding_window is not None,
        }
        if self.sliding_window is not None:
            d["sliding_window"] = self.sliding_window
            d["layer_types"] = list(self.layer_types)
        return d

    # ------------------------------------------------------------------ the parts of each layer
    def model_spec(self) -> ModelSpec:
        """Pre-norm blocks of grouped-query attention (per-head q/k RMSNorm, then rotate-half
        RoPE) and a SwiGLU feed-forward; final RMSNorm; tied or untied output head
        (``engine/dryft_qwen3/model.py:122-187``)."""
        norm = PartSpec("rmsnorm", {"size": self.hidden_size, "eps": self.rms_norm_eps})
        layers = []
        types = self.layer_types or tuple(FULL_ATTENTION for _ in range(self.num_hidden_layers))
        for i in range(self.num_hidden_layers):
            window = self.sliding_window if types[i] == SLIDING_ATTENTION else None
            mixer = PartSpec(
                "attention",
                {
                    "hidden_size": self.hidden_size,
                    "num_heads": self.num_attention_heads,
                    "num_kv_heads": self.num_key_value_heads,
                    "head_dim": self.head_dim,
                    "scale": self.attention_scale,
                    "window": window,
                    "qk_norm": PartSpec("rmsnorm", {"size": self.head_dim, "eps": self.rms_norm_eps}),
                    "position": PartSpec("rope", {"rotary_dim": self.head_dim, "theta": self.rope_theta}),
                },
            )
            ffn = PartSpec(
                "swiglu",
                {"hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size},
            )
            layers.append(
                LayerSpec(
                    block="prenorm",
                    mixer=mixer,
                    ffn=ffn,
                    norm_mixer=norm,
                    norm_ffn=norm,
                    mixer_prefix=f"model.layers.{i}.self_attn.",
                    ffn_prefix=f"model.layers.{i}.mlp.",
                    norm_mixer_prefix=f"model.layers.{i}.input_layernorm.",
                    norm_ffn_prefix=f"model.layers.{i}.post_attention_layernorm.",
                )
            )
        spec = ModelSpec(
            architecture=self.architecture,
            vocab_size=self.vocab_size,
            hidden_size=self.hidden_size,
            max_positions=self.max_position_embeddings,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size}),
            layers=tuple(layers),
            schedule=tuple(RunStep(layer=i) for i in range(self.num_hidden_layers)),
            final_norm=norm,
            head=PartSpec(
                "lm_head",
                {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size, "tied": self.tie_word_embeddings},
            ),
        )
        spec.validate()
        return spec
