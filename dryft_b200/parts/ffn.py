"""SwiGLU feed-forward: ``down(silu(gate(h)) * up(h))`` with gate and up fused into one product
``[rows, 2I]`` (gate columns first; ``engine/dryft_qwen3/weights.py:98-100``; ``model.py:180``), the
silu rounded to the activation dtype before it multiplies up (``kernels/silu_mul.py:29-32``).
Rows are independent, so long prompts go through in chunks that bound the ``[rows, 2I]`` product.
"""

from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..ops import kernels as K
from .base import Runtime, StepContext, TensorInfo, register_ffn
from .linear import linear


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
