"""``y = x @ W.T`` for the weights of the parts (all ``[out, in]``, no bias — ``OPTIMIZATION_GUIDE.md:117``;
``engine/dryft_qwen3/config.py:138``).

Which product runs:
  * 32-bit activations (the 32-bit path): the hand-written CUDA-core product, true fp32;
  * bfloat16, few rows (decode): the hand-written weight-streaming tensor-core products -- through registers into
    mma.sync up to ``small_m_max`` rows, by TMA into tcgen05.mma up to ``stream_m_max`` (64);
  * bfloat16, many rows (prefill): cuBLAS through ``torch.mm``, 32-bit accumulation — the library
    product the reference itself uses (``F.linear``, ``engine/dryft_qwen3/model.py:153,179,180``);
  * bfloat16 activations with a weight the checkpoint stores in 32-bit: the weight stays 32-bit,
    the activations are widened, the 32-bit product runs and its result is rounded once.
"""

from __future__ import annotations

from typing import Optional

import torch

from ..ops import kernels as K
from .base import Runtime, fused_rms


def linear(x: torch.Tensor, w: torch.Tensor, rt: Runtime, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    out_dtype = out_dtype or x.dtype
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise ValueError(f"linear: activations have width {k}, weight is {tuple(w.shape)}")
    if x.dtype == torch.float32:
        if w.dtype != torch.float32:
            raise ValueError(f"linear: 32-bit activations need a 32-bit weight, got {w.dtype}")
        out = torch.empty((m, n), dtype=torch.float32, device=x.device)
        K.gemm_nt_f32(x, w, out)
        return out if out_dtype == torch.float32 else out.to(out_dtype)
    if x.dtype != torch.bfloat16:
        raise ValueError(f"linear: activations are float32 or bfloat16, got {x.dtype}")
    if w.dtype == torch.float32:
        out = torch.empty((m, n), dtype=torch.float32, device=x.device)
        K.gemm_nt_f32(x.to(torch.float32), w, out)
        return out if out_dtype == torch.float32 else out.to(out_dtype)
    if w.dtype != torch.bfloat16:
        raise ValueError(f"linear: weight dtype {w.dtype} is not supported")
    if K.fused_rows_supported(m, k, rt.small_m_max, 0, normed=True):   # above 8 rows: the narrow widths only
        out = torch.empty((m, n), dtype=out_dtype, device=x.device)
        K.gemm_small_m(x, w, out)
        return out
    if m <= min(rt.stream_m_max, K.STREAM_M_LIMIT) and K.gemm_stream_supported(m, k) and rt.tcgen05:
        out = torch.empty((m, n), dtype=out_dtype, device=x.device)
        K.gemm_stream(x, w, out)
        return out
    if out_dtype == torch.bfloat16:
        return torch.mm(x, w.t())
    return torch.mm(x, w.t(), out_dtype=out_dtype)


def fusable_rows(n_rows: int, k: int, rt: Runtime, normed: bool = False) -> bool:
    """Whether the fused decode products take ``n_rows`` rows over ``k`` inputs (``normed``: with a norm on the way in)."""
    return K.fused_rows_supported(n_rows, k, rt.small_m_max, rt.stream_m_max if rt.tcgen05 else 0, normed)


def weighted_for(next_norm, width: int, k_in: int, rt: Runtime, n_rows: int = 1) -> bool:
    """Whether a fused decode product of ``k_in`` inputs that updates a stream of ``width`` should also leave
    the stream weighted for ``next_norm`` (an RMS norm over ``width``): both it and the product behind that
    norm must be of the form compiled per inner size (which takes up to ``small_m_max`` rows)."""
    rms = fused_rms(next_norm) if next_norm is not None else None
    return (rms is not None and rt.norm_ahead and rt.is_bf16 and rms[0].numel() == width
            and n_rows <= min(rt.small_m_max, K.SMALL_M_LIMIT)
            and K.weighted_ahead_supported(width) and K.weighted_ahead_supported(k_in))
