"""Named ``config.json`` contents: the two tiny test configurations and the three
benchmark shapes.  These are data fed to ``config_from_dict`` exactly as a model
folder's ``config.json`` would be; nothing else in the package refers to them.

The tiny shape follows ``agent/verify.py:36-54`` (2 layers, width 64, 4/2 heads,
head size 16, intermediate 128, vocabulary 256, tied); the second tiny shape differs
from it in every size and option.  The 4B shape is the checkpoint the reference pins
(``engine/dryft_qwen3/config.py:55-70``).
"""

from __future__ import annotations


def _qwen3(**kw) -> dict:
    base = {
        "architectures": ["Qwen3ForCausalLM"],
        "model_type": "qwen3",
        "hidden_act": "silu",
        "attention_bias": False,
        "rope_scaling": None,
        "use_sliding_window": False,
    }
    base.update(kw)
    return base


PRESETS = {
    "tiny-a": _qwen3(
        num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
        intermediate_size=128, vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6,
        tie_word_embeddings=True, max_position_embeddings=128,
    ),
    "tiny-b": _qwen3(
        num_hidden_layers=3, hidden_size=80, num_attention_heads=6, num_key_value_heads=3, head_dim=32,
        intermediate_size=224, vocab_size=384, rope_theta=1000000.0, rms_norm_eps=1e-5,
        tie_word_embeddings=False, max_position_embeddings=256,
    ),
    "qwen3-4b": _qwen3(
        num_hidden_layers=36, hidden_size=2560, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
        intermediate_size=9728, vocab_size=151936, rope_theta=5000000.0, rms_norm_eps=1e-6,
        tie_word_embeddings=True, max_position_embeddings=8192,
    ),
    "qwen3-8b": _qwen3(
        num_hidden_layers=36, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
        intermediate_size=12288, vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6,
        tie_word_embeddings=False, max_position_embeddings=8192,
    ),
    "qwen3-32b": _qwen3(
        num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, num_key_value_heads=8, head_dim=128,
        intermediate_size=25600, vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6,
        tie_word_embeddings=False, max_position_embeddings=16384,
    ),
}


def preset(name: str) -> dict:
    if name not in PRESETS:
        raise KeyError(f"unknown preset {name!r}; known: " + ", ".join(sorted(PRESETS)))
    return dict(PRESETS[name])
