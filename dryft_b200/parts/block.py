"""Arrangements of a mixer, a feed-forward and their norms in one layer.

``prenorm`` (``engine/dryft_qwen3/model.py:151-184``):
    x += delta_in ; h = norm_mixer(x)          (one fused kernel; delta_in is the previous block's
    a  = mixer(h)                               not-yet-added feed-forward output)
    x += a        ; h = norm_ffn(x)            (one fused kernel)
    delta_out = ffn(h)
The block returns ``(x, delta_out)``: the add of ``delta_out`` is left to whatever norm comes next (the
next block's, or the final norm), which is how the reference fuses "residual add + next norm".
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from .base import StepContext, register_block


@register_block("prenorm")
class PreNormBlock:
    def __init__(self, norm_mixer, mixer, norm_ffn, ffn):
        self.norm_mixer = norm_mixer
        self.mixer = mixer
        self.norm_ffn = norm_ffn
        self.ffn = ffn

    def forward(self, x: torch.Tensor, delta: Optional[torch.Tensor], ctx: StepContext, cache, state,
                owns_cache: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
        h = self.norm_mixer.forward(x) if delta is None else self.norm_mixer.add_forward(x, delta)
        a = self.mixer.forward(h, ctx, cache, state, owns_cache)
        h = self.norm_ffn.add_forward(x, a)
        return x, self.ffn.forward(h, ctx)
