"""Position encodings a mixer can be given.

``rope``: rotate-half rotary embedding (``engine/dryft_qwen3/model.py:35-41,49-57``):
``inv_freq[j] = 1 / theta^(2j/R)`` for ``j = 0..R/2-1`` from ``arange(0, R, 2)`` int64 -> float32, angle
``pos * inv_freq[j]`` in 32-bit, cos/sin cast to the activation dtype, dims ``j`` and ``j + R/2``
rotated together.  ``R`` (``rotary_dim``) may be smaller than the head size.  The angles and their
cos/sin are evaluated on the device (``csrc/rope_kv.cu``) from the position of each token: inside the
fused kernels for a decode step, and once per step into a table that all layers with the same
``(theta, rotary_dim)`` share for a step of many tokens.  This part owns ``inv_freq``, computed on the
host with exactly the reference's expression so that the 32-bit products ``pos * inv_freq`` agree bit
for bit with a table built the reference's way.

``none``: no position encoding (``rotary_dim = 0``).
"""

from __future__ import annotations

from typing import Mapping, Optional

import torch

from ..ops import kernels as K
from .base import Runtime, StepContext, register_position

TABLE_MIN_TOKENS = 64   # below this every warp evaluates its own angles


@register_position("rope")
class Rope:
    def __init__(self, params: Mapping, head_dim: int, rt: Runtime):
        self.rotary_dim = int(params.get("rotary_dim", head_dim))
        self.theta = float(params["theta"])
        if self.rotary_dim <= 0 or self.rotary_dim % 2 or self.rotary_dim > head_dim:
            raise ValueError(f"rope: rotary_dim must be even and in (0, head_dim={head_dim}], got {self.rotary_dim}")
        r = self.rotary_dim
        inv_freq = 1.0 / (self.theta ** (torch.arange(0, r, 2, dtype=torch.int64).to(torch.float32) / r))
        self.inv_freq: Optional[torch.Tensor] = inv_freq.to(rt.device)
        self.dtype = rt.dtype

    def table(self, ctx: StepContext) -> Optional[torch.Tensor]:
        """The step's cos / sin table, made by the first layer that asks and kept in the step's context."""
        if ctx.decode or ctx.n_tokens < TABLE_MIN_TOKENS:
            return None
        key = ("rope_table", self.theta, self.rotary_dim)
        table = ctx.extras.get(key)
        if table is None:
            table = K.rope_table(ctx.tok_pos, self.inv_freq, ctx.n_tokens, self.dtype)
            ctx.extras[key] = table
        return table


@register_position("none")
class NoPosition:
    def __init__(self, params: Mapping, head_dim: int, rt: Runtime):
        self.rotary_dim = 0
        self.inv_freq = None

    def table(self, ctx: StepContext) -> None:
        return None
