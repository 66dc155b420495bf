"""Token choice: greedy, temperature and top-k.

hari495/dryft is greedy only: ``argmax`` of the last position's logits, the first index on ties
(``engine/dryft_qwen3/model.py:187,262``; ``AGENTS.md:174-175``).  Here ``temperature == 0`` is that
argmax over the 32-bit logits; otherwise the ``top_k`` largest logits are kept (0 keeps all), divided
by the temperature, soft-maxed in 32-bit and drawn from with a counter-based uniform keyed by
``(seed, sequence index, step)`` — so a sequence's draws do not depend on its slot, on the batch it
runs in, or on how many sequences ran before it.  The kernels are in ``csrc/sample.cu``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..ops import kernels as K


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0
    seed: int = 0

    def __post_init__(self):
        if self.temperature < 0.0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if self.top_k < 0:
            raise ValueError(f"top_k must be >= 0, got {self.top_k}")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0


def choose(logits: torch.Tensor, params: SamplingParams, *, row_seq: Optional[torch.Tensor] = None, step: int = 0,
           row_slot: Optional[torch.Tensor] = None, last_token: Optional[torch.Tensor] = None,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of ``logits`` ``[rows, vocab]`` (float32, on the device) -> int32 ``[rows]``.
    Row ``r`` belongs to sequence ``row_seq[r]`` (``r`` if None) and is at generation step ``step``.
    With ``row_slot`` and ``last_token`` the choice is also recorded in the per-sequence state."""
    rows = logits.shape[0]
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    if params.greedy:
        K.argmax_rows(logits, out, row_slot, last_token)
    else:
        K.sample_rows(logits, params.temperature, params.top_k, params.seed, row_seq, None, out, row_slot, last_token,
                      step_base=step)
    return out
