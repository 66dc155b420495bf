"""Arrangements of a mixer, a feed-forward and their norms in one layer.

``prenorm`` (``engine/dryft_qwen3/model.py:151-184``):
    x += delta_in ; h = norm_mixer(x)          (one fused kernel; delta_in is the previous block's
    a  = mixer(h)                               not-yet-added feed-forward output)
    x += a        ; h = norm_ffn(x)            (one fused kernel)
    delta_out = ffn(h)
The block returns the stream and ``delta_out``: the add of ``delta_out`` is left to whatever norm comes
next (the next block's, or the final norm), which is how the reference fuses "residual add + next
norm".  With few rows (decode) and parts that offer it, the norms, the adds and the activation are
folded into the matrix products instead (``csrc/gemm_small_m.cu``).
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from ..ops import kernels as K
from .base import Residual, StepContext, register_block


@register_block("prenorm")
class PreNormBlock:
    def __init__(self, norm_mixer, mixer, norm_ffn, ffn):
        self.norm_mixer = norm_mixer
        self.mixer = mixer
        self.norm_ffn = norm_ffn
        self.ffn = ffn

    def _fusable(self, n_rows: int) -> bool:
        m, f = self.mixer, self.ffn
        return (hasattr(m, "forward_normed") and hasattr(f, "forward_normed")
                and m.can_fuse(n_rows, self.norm_mixer) and f.can_fuse(n_rows, self.norm_ffn))

    def forward(self, res: Residual, ctx: StepContext, cache, state, owns_cache: bool = True) -> Residual:
        x = res.x
        if self._fusable(x.shape[0]):
            # few rows: five launches per layer.  Each product normalises / adds / activates on its own
            # and hands the stream's sums of squares to the next one.
            if res.delta is not None:
                K.residual_add(x, res.delta)
                res = Residual(x)
            ss, parts = res.ss, res.ss_parts
            if ss is None:
                ss = torch.empty(K.SS_STRIDE, dtype=torch.float32, device=x.device)
                K.row_sumsq(x, ss)
                parts = 1
            ss, parts = self.mixer.forward_normed(x, ss, parts, self.norm_mixer, ctx, cache, state, owns_cache)
            ss, parts = self.ffn.forward_normed(x, ss, parts, self.norm_ffn, ctx)
            return Residual(x, None, ss, parts)
        h = self.norm_mixer.forward(x) if res.delta is None else self.norm_mixer.add_forward(x, res.delta)
        a = self.mixer.forward(h, ctx, cache, state, owns_cache)
        h = self.norm_ffn.add_forward(x, a)
        return Residual(x, self.ffn.forward(h, ctx))
