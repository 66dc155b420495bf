"""RMSNorm: ``w * cast(x32 * rsqrt(mean(x32^2) + eps))`` — the weight multiplies after the cast
back to the activation dtype, and ``(1 + w)`` is not used (``engine/dryft_qwen3/model.py:28-32``;
``kernels/rmsnorm.py:3-6,36-39``).  Its weight is kept in 32-bit on the device (an exact widening of
a bfloat16 tensor) so one kernel serves both precisions.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..ops import kernels as K
from .base import Runtime, TensorInfo, register_norm


@register_norm("rmsnorm")
class RMSNorm:
    @staticmethod
    def tensors(params: Mapping, prefix: str) -> Dict[str, TensorInfo]:
        return {prefix + "weight": TensorInfo((params["size"],), "vector")}

    def __init__(self, params: Mapping, prefix: str, weights, rt: Runtime):
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.rt = rt
        self.weight = weights.load(prefix + "weight", "vector")  # float32 [size]

    def rms_params(self):
        """This norm is ``weight * cast(x32 * rsqrt(mean(x32^2) + eps))``: products may fold it into themselves."""
        return self.weight, self.eps

    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None) -> torch.Tensor:
        n = n_rows if n_rows is not None else (rows.numel() if rows is not None else x.shape[0])
        out = torch.empty((n, self.size), dtype=x.dtype, device=x.device)
        K.rmsnorm(x, self.weight, self.eps, out, rows=rows)
        return out

    def add_forward(self, x: torch.Tensor, delta: torch.Tensor, rows: Optional[torch.Tensor] = None,
                    n_rows: Optional[int] = None) -> torch.Tensor:
        """``x += delta`` (32-bit sum, rounded once) and the norm of the sum.  With ``rows`` only those
        rows are summed and normed, and ``x`` is left as it is."""
        n = n_rows if n_rows is not None else (rows.numel() if rows is not None else x.shape[0])
        out = torch.empty((n, self.size), dtype=x.dtype, device=x.device)
        K.rmsnorm(x, self.weight, self.eps, out, delta=delta, rows=rows, x_out=None if rows is not None else x)
        return out
