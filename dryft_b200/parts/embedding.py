"""Token embedding ``x = embed[ids]`` (``engine/dryft_qwen3/model.py:132,226``) and the output head
``logits = h @ W_head.T`` with ``W_head`` the embedding table itself when tied
(``engine/dryft_qwen3/weights.py:47-49``).  Unlike the reference, an untied ``lm_head.weight`` is
served (``weights.py:84-85`` refuses it), and logits leave the product's 32-bit accumulator
unrounded.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..ops import kernels as K
from .base import Runtime, TensorInfo, fused_rms, register_embedding, register_head
from .linear import fusable_rows, linear


@register_embedding("embedding")
class Embedding:
    @staticmethod
    def tensors(params: Mapping, prefix: str) -> Dict[str, TensorInfo]:
        return {prefix + "weight": TensorInfo((params["vocab_size"], params["hidden_size"]), "table")}

    def __init__(self, params: Mapping, prefix: str, weights, rt: Runtime):
        self.rt = rt
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.table = weights.load(prefix + "weight", "table")
        # raised by the gather for an id outside the table (its row is zeroed, not read); read with the other
        # device flags by ``kernels.check_error_flags``
        self.err = torch.zeros(1, dtype=torch.int32, device=rt.device)
        K.watch_flag(self.err, "a token id outside the embedding table reached the embedding gather (its row was zeroed)")

    def forward(self, tokens: torch.Tensor, n_rows: int) -> torch.Tensor:
        out = torch.empty((n_rows, self.hidden), dtype=self.table.dtype, device=self.table.device)
        K.embed(tokens, self.table, out, self.err)
        # a table the checkpoint stores in 32-bit stays 32-bit; its rows are rounded on the way out
        return out if out.dtype == self.rt.dtype else out.to(self.rt.dtype)


@register_head("lm_head")
class LMHead:
    @staticmethod
    def tensors(params: Mapping, prefix: str) -> Dict[str, TensorInfo]:
        return {prefix + "weight": TensorInfo((params["vocab_size"], params["hidden_size"]), "matrix",
                                        optional=bool(params["tied"]))}

    def __init__(self, params: Mapping, prefix: str, weights, rt: Runtime, embedding: Optional[Embedding] = None):
        self.rt = rt
        self.vocab = int(params["vocab_size"])
        self.tied = bool(params["tied"])
        name = prefix + "weight"
        if self.tied:
            if embedding is None:
                raise ValueError("a tied output head needs the embedding it is tied to")
            self.weight = embedding.table
            if weights.has(name):
                # present although tied: it has to be the same tensor (weights.py:86-87)
                other = weights.load(name, "matrix")
                if other.shape != self.weight.shape or not torch.equal(other.to(self.weight.dtype), self.weight):
                    raise ValueError(f"{name} is present and differs from the embedding table although the "
                                     "output head is tied to it")
                del other
        else:
            self.weight = weights.load(name, "matrix")

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        """32-bit logits ``[rows, vocab]``."""
        return linear(h, self.weight, self.rt, out_dtype=torch.float32)

    def can_fuse(self, n_rows: int, norm) -> bool:
        rt = self.rt
        return (rt.fuse_decode and rt.is_bf16 and fusable_rows(n_rows, self.weight.shape[1], rt, normed=True)
                and fused_rms(norm) is not None and self.weight.dtype == torch.bfloat16)

    def forward_normed(self, x: torch.Tensor, ss, ss_parts: int, norm, xw=None) -> torch.Tensor:
        """Logits of every row of ``x`` with the final norm inside the product (decode); ``xw``: ``x``
        weighted by the final norm's weight already."""
        out = torch.empty((x.shape[0], self.vocab), dtype=torch.float32, device=x.device)
        norm_w, eps = fused_rms(norm)
        small = self.rt.small_m_max
        if xw is not None and K.weighted_ahead_supported(x.shape[1]):
            K.fused_product(x, self.weight, out, small_m_max=small, xw_in=xw, norm_w=norm_w, ss_in=ss, ss_parts=ss_parts, eps=eps, pdl=self.rt.pdl)
        else:
            K.fused_product(x, self.weight, out, small_m_max=small, norm_w=norm_w, ss_in=ss, ss_parts=ss_parts, eps=eps, pdl=self.rt.pdl)
        return out
