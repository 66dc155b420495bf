"""dryft_b200 — a small, whole, single-GPU generation library for the Qwen3 dense decoder,
written for NVIDIA B200 (sm_100a): everything between a request's tokens and its next token.

    from dryft_b200 import Engine
    eng = Engine(model_dir)                       # config.json + model.safetensors
    for step in eng.generate([[1, 2, 3], [4, 5]], max_new_tokens=8):
        print(step)                               # one token id per sequence

The entry point mirrors ``engine/engine.py:28-30,138-140`` of hari495/dryft.
"""

__version__ = "0.1.0"


def __getattr__(name):
    if name in ("Engine", "EngineOptions"):
        from .engine import api

        return getattr(api, name)
    raise AttributeError(name)
