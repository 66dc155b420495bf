"""SwiGLU feed-forward: ``down(silu(gate(h)) * up(h))`` with gate and up fused into one product
``[rows, 2I]`` (gate columns first; ``engine/dryft_qwen3/weights.py:98-100``; ``model.py:180``), the
silu rounded to the activation dtype before it multiplies up (``kernels/silu_mul.py:29-32``).
Rows are independent, so long prompts go through in chunks that bound the ``[rows, 2I]`` product.
"""

from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..ops import kernels as K
from .base import Runtime, StepContext, TensorInfo, fused_rms, register_ffn
from .linear import fusable_rows, linear, weighted_for


@register_ffn("swiglu")
class SwiGLU:
    @staticmethod
    def tensors(params: Mapping, prefix: str) -> Dict[str, TensorInfo]:
        h, i = params["hidden_size"], params["intermediate_size"]
        return {
            prefix + "gate_proj.weight": TensorInfo((i, h), "matrix"),
            prefix + "up_proj.weight": TensorInfo((i, h), "matrix"),
            prefix + "down_proj.weight": TensorInfo((h, i), "matrix"),
        }

    def __init__(self, params: Mapping, prefix: str, weights, rt: Runtime):
        self.rt = rt
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.w_gate_up = weights.load_fused(
            [prefix + "gate_proj.weight", prefix + "up_proj.weight"], [self.inter, self.inter], self.hidden)
        self.w_down = weights.load(prefix + "down_proj.weight", "matrix")

    def can_fuse(self, n_rows: int, norm) -> bool:
        rt = self.rt
        return (rt.fuse_decode and rt.is_bf16 and fusable_rows(n_rows, self.hidden, rt, normed=True) and fusable_rows(n_rows, self.inter, rt)
                and fused_rms(norm) is not None and self.w_gate_up.dtype == torch.bfloat16 and self.w_down.dtype == torch.bfloat16)

    weighted_ahead = True   # forward_normed takes ``xw`` / ``next_norm`` and returns the weighted stream too

    def forward_normed(self, x, ss, ss_parts, norm, ctx, xw=None, next_norm=None):
        """``x += down(silu(gate(norm(x))) * up(norm(x)))`` in place, two launches: the norm and the
        SiLU*mul inside the first product, the add (and the new sums of squares) inside the second.
        ``xw`` / ``next_norm`` as in the attention mixer.  Returns ``(ss, ss_parts, xw or None)``."""
        n = x.shape[0]
        act = torch.empty((n, self.inter), dtype=x.dtype, device=x.device)
        norm_w, eps = fused_rms(norm)
        small = self.rt.small_m_max
        if xw is not None and K.weighted_ahead_supported(self.hidden):
            K.fused_product(x, self.w_gate_up, act, small_m_max=small, mode="silu", xw_in=xw, norm_w=norm_w, ss_in=ss, ss_parts=ss_parts,
                            eps=eps, pdl=self.rt.pdl)
        else:
            K.fused_product(x, self.w_gate_up, act, small_m_max=small, mode="silu", norm_w=norm_w, ss_in=ss, ss_parts=ss_parts, eps=eps,
                            pdl=self.rt.pdl)
        parts = K.fused_ss_parts(n, self.hidden, self.inter, small)
        ss_out = torch.empty(parts * K.SS_STRIDE, dtype=torch.float32, device=x.device)
        xw_out = None
        if weighted_for(next_norm, self.hidden, self.inter, self.rt, n):
            xw_out = torch.empty_like(x)
            K.fused_product(act, self.w_down, x, small_m_max=small, mode="residual", ss_out=ss_out, pdl=self.rt.pdl,
                            next_w=fused_rms(next_norm)[0], xw_out=xw_out)
        else:
            K.fused_product(act, self.w_down, x, small_m_max=small, mode="residual", ss_out=ss_out, pdl=self.rt.pdl)
        return ss_out, parts, xw_out

    def _rows(self, h: torch.Tensor) -> torch.Tensor:
        gu = linear(h, self.w_gate_up, self.rt)
        act = torch.empty((h.shape[0], self.inter), dtype=h.dtype, device=h.device)
        K.silu_mul(gu, act)
        return linear(act, self.w_down, self.rt)

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        n = h.shape[0]
        chunk = self.rt.ffn_chunk_rows
        if n <= chunk:
            return self._rows(h)
        out = torch.empty((n, self.hidden), dtype=h.dtype, device=h.device)
        for r0 in range(0, n, chunk):
            out[r0:r0 + chunk] = self._rows(h[r0:r0 + chunk])
        return out
