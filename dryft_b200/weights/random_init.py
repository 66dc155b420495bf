"""Random-weights mode: write a model folder (``config.json`` + ``model.safetensors``) from a
configuration and a seed.

Matrices and the embedding are ``normal(0, std)``, norm weights ``1 + normal(0, std)``, drawn in
float32 on the CPU from a generator seeded by (seed, tensor name), then stored in ``dtype``.  A tied
model stores no ``lm_head.weight``.  (The reference's tooling makes its tiny model with another
library and multiplies its weights by 4 so that logits are not flat, ``agent/verify.py:36-54``;
``std`` plays that role here.)
"""

from __future__ import annotations

import json
import os
from typing import Any, Dict, Mapping, Union

import torch
from safetensors.torch import save_file

from ..config import config_from_dict
from .expected import expected_tensors
from .source import random_tensor


def random_state_dict(config: Any, seed: int, dtype: torch.dtype = torch.bfloat16, std: float = 0.02) -> Dict[str, torch.Tensor]:
    spec = config.model_spec()
    out: Dict[str, torch.Tensor] = {}
    for name, info in expected_tensors(spec).items():
        if info.optional:  # a tied output head is not stored
            continue
        out[name] = random_tensor(name, info, seed, std, torch.device("cpu")).to(dtype).contiguous()
    return out


def write_random_model(config: Union[Mapping[str, Any], Any], seed: int, out_dir: str,
                       dtype: torch.dtype = torch.bfloat16, std: float = 0.02) -> str:
    """``config`` is a config.json mapping or a typed configuration.  Returns ``out_dir``."""
    cfg = config_from_dict(config) if isinstance(config, Mapping) else config
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg.to_dict(), f, indent=1)
    save_file(random_state_dict(cfg, seed, dtype, std), os.path.join(out_dir, "model.safetensors"),
              metadata={"format": "pt"})
    return out_dir
