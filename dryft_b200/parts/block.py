"""Arrangements of a mixer, a feed-forward and their norms in one layer.

``prenorm`` (``engine/dryft_qwen3/model.py:151-184``):
    x += delta_in ; h = norm_mixer(x)          (one fused kernel; delta_in is the previous block's
    a  = mixer(h)                               not-yet-added feed-forward output)
    x += a        ; h = norm_ffn(x)            (one fused kernel)
    delta_out = ffn(h)
A layer without a feed-forward stops after the mixer and returns its output as ``delta_out``.
The block returns the stream and ``delta_out``: the add of ``delta_out`` is left to whatever norm comes
next (the next block's, or the final norm), which is how the reference fuses "residual add + next
norm".  With few rows (decode) and parts that offer it, the norms, the adds and the activation are
folded into the matrix products instead (``csrc/gemm_small_m.cu``).
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from ..ops import kernels as K
from .base import Residual, StepContext, fused_rms, register_block
from .linear import weighted_for


@register_block("prenorm")
class PreNormBlock:
    def __init__(self, norm_mixer, mixer, norm_ffn, ffn):
        self.norm_mixer = norm_mixer
        self.mixer = mixer
        self.norm_ffn = norm_ffn
        self.ffn = ffn

    def _fusable(self, n_rows: int) -> bool:
        m, f = self.mixer, self.ffn
        if f is None:
            return False
        return (hasattr(m, "forward_normed") and hasattr(f, "forward_normed")
                and m.can_fuse(n_rows, self.norm_mixer) and f.can_fuse(n_rows, self.norm_ffn))

    takes_next_norm = True   # forward accepts the norm that will read the stream after this block

    def forward(self, res: Residual, ctx: StepContext, cache, state, owns_cache: bool = True, next_norm=None) -> Residual:
        x = res.x
        if self._fusable(x.shape[0]):
            # few rows: five launches per layer.  Each product normalises / adds / activates on its own
            # and hands the stream's sums of squares (and, where sizes allow, the stream weighted for the
            # next norm) to the next one.
            if res.delta is not None:
                K.residual_add(x, res.delta)
                res = Residual(x)
            ss, parts = res.ss, res.ss_parts
            xw = res.xw if res.xw_norm is self.norm_mixer else None
            ahead_m = getattr(self.mixer, "weighted_ahead", False)
            ahead_f = getattr(self.ffn, "weighted_ahead", False)
            if ss is None:
                ss = torch.empty(K.SS_STRIDE, dtype=torch.float32, device=x.device)
                if ahead_m and weighted_for(self.norm_mixer, x.shape[1], x.shape[1], self.mixer.rt, x.shape[0]):
                    xw = torch.empty_like(x)
                    K.row_sumsq(x, ss, norm_w=fused_rms(self.norm_mixer)[0], xw_out=xw)
                else:
                    K.row_sumsq(x, ss)
                parts = 1
            if ahead_m:
                ss, parts, xw = self.mixer.forward_normed(x, ss, parts, self.norm_mixer, ctx, cache, state, owns_cache,
                                                          xw=xw, next_norm=self.norm_ffn if ahead_f else None)
            else:
                ss, parts = self.mixer.forward_normed(x, ss, parts, self.norm_mixer, ctx, cache, state, owns_cache)
                xw = None
            if ahead_f:
                ss, parts, xw = self.ffn.forward_normed(x, ss, parts, self.norm_ffn, ctx, xw=xw, next_norm=next_norm)
            else:
                ss, parts = self.ffn.forward_normed(x, ss, parts, self.norm_ffn, ctx)
                xw = None
            return Residual(x, None, ss, parts, xw, next_norm if xw is not None else None)
        h = self.norm_mixer.forward(x) if res.delta is None else self.norm_mixer.add_forward(x, res.delta)
        a = self.mixer.forward(h, ctx, cache, state, owns_cache)
        if self.ffn is None:           # a layer without a feed-forward: the mixer's output is what the next norm adds
            return Residual(x, a)
        h = self.norm_ffn.add_forward(x, a)
        return Residual(x, self.ffn.forward(h, ctx))
