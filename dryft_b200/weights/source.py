"""Where parts get their tensors from: a checkpoint, or a seeded random generator.

Precision on the device (``resolve_dtype``):
  * the 32-bit path widens everything to float32 (exact);
  * the bfloat16 path keeps bfloat16 tensors as they are; a tensor the checkpoint stores in 32-bit
    stays 32-bit (the product then runs in 32-bit for that weight); float16 is converted to bfloat16;
  * 1-D tensors (norm weights) are kept in float32 in both paths — for a bfloat16 tensor that is an
    exact widening, and one norm kernel serves both;
  * integer tensors become int32.
The reference casts every tensor to bfloat16 (``engine/dryft_qwen3/weights.py:76-78``).
"""

from __future__ import annotations

import hashlib
from typing import Dict, List, Mapping, Optional, Sequence

import torch

from ..parts.base import TensorInfo
from .checkpoint import Checkpoint, WeightsError


def resolve_dtype(stored: torch.dtype, engine: torch.dtype, kind: str) -> torch.dtype:
    if not stored.is_floating_point:
        return torch.int32
    if engine == torch.float32 or kind == "vector":
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


class WeightSource:
    """Interface the parts load through."""

    engine_dtype: torch.dtype
    device: torch.device

    def has(self, name: str) -> bool:
        raise NotImplementedError

    def stored_dtype(self, name: str) -> torch.dtype:
        raise NotImplementedError

    def _read(self, name: str) -> torch.Tensor:
        """The stored tensor, on any device."""
        raise NotImplementedError

    def load(self, name: str, kind: str) -> torch.Tensor:
        t = self._read(name)
        dt = resolve_dtype(t.dtype, self.engine_dtype, kind)
        return t.to(device=self.device, dtype=dt).contiguous()

    def load_fused(self, names: Sequence[str], rows: Sequence[int], cols: int) -> torch.Tensor:
        """Rows of several matrices stacked into one (q;k;v and gate;up —
        ``engine/dryft_qwen3/weights.py:93-100``), read one at a time into the final buffer."""
        dts = {resolve_dtype(self.stored_dtype(n), self.engine_dtype, "matrix") for n in names}
        dt = dts.pop() if len(dts) == 1 else torch.float32
        out = torch.empty((sum(rows), cols), dtype=dt, device=self.device)
        r0 = 0
        for n, r in zip(names, rows):
            t = self._read(n)
            if tuple(t.shape) != (r, cols):
                raise WeightsError("fused load", [], [], [(n, (r, cols), tuple(t.shape))])
            out[r0:r0 + r].copy_(t.to(device=self.device, dtype=dt))
            r0 += r
        return out


class CheckpointSource(WeightSource):
    def __init__(self, checkpoint: Checkpoint, engine_dtype: torch.dtype, device: torch.device):
        self.ckpt = checkpoint
        self.engine_dtype = engine_dtype
        self.device = device

    def has(self, name: str) -> bool:
        return self.ckpt.has(name)

    def stored_dtype(self, name: str) -> torch.dtype:
        return self.ckpt.dtypes[name]

    def _read(self, name: str) -> torch.Tensor:
        return self.ckpt.read(name)


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def random_tensor(name: str, info: TensorInfo, seed: int, std: float, device: torch.device) -> torch.Tensor:
    """float32 values of one tensor: matrices and tables ``normal(0, std)``, vectors (norm weights)
    ``1 + normal(0, std)``.  Each tensor has its own generator seeded from (seed, name), so the
    values do not depend on the order tensors are asked for.  (The reference only has random
    weights through its tooling, ``agent/verify.py:36-54``.)"""
    gen = torch.Generator(device=device)
    gen.manual_seed(_tensor_seed(seed, name))
    t = torch.randn(info.shape, generator=gen, dtype=torch.float32, device=device) * std
    if info.kind == "vector":
        t += 1.0
    return t


class RandomSource(WeightSource):
    """Random weights without a model folder, values rounded to ``store_dtype`` first as a checkpoint
    would hold them."""

    def __init__(self, expected: Mapping[str, TensorInfo], seed: int, engine_dtype: torch.dtype, device: torch.device,
                 std: float = 0.02, store_dtype: torch.dtype = torch.bfloat16, skip: Sequence[str] = (),
                 draw_device: Optional[torch.device] = None):
        # the generator the values come from: the device's by default; the CPU's gives the very tensors that
        # ``write_random_model`` stores for the same seed (the two generators differ)
        self.draw_device = draw_device if draw_device is not None else device
        self.expected = dict(expected)
        self.seed = seed
        self.std = std
        self.engine_dtype = engine_dtype
        self.device = device
        self.store_dtype = store_dtype
        self.skip = set(skip)

    def has(self, name: str) -> bool:
        return name in self.expected and name not in self.skip

    def stored_dtype(self, name: str) -> torch.dtype:
        return self.store_dtype

    def _read(self, name: str) -> torch.Tensor:
        return random_tensor(name, self.expected[name], self.seed, self.std, self.draw_device).to(self.store_dtype)
