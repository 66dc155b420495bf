"""Reading a model folder's safetensors by tensor name.

File discovery follows ``engine/dryft_qwen3/weights.py:52-61``: ``model.safetensors.index.json`` names
the shards, else every ``*.safetensors`` in the folder.  Unlike the reference (which loads the whole
checkpoint to the device and then fuses, ``weights.py:66-70,96-101``), tensors are read one at a time
into buffers of their final shape, and the whole name/shape comparison happens before anything is
loaded: ONE error lists every missing tensor, every unexpected tensor and every wrong shape
(the reference stops at the first, ``weights.py:73-75``, and only warns about leftovers, ``:115-116``).
"""

from __future__ import annotations

import glob
import json
import os
from typing import Dict, List, Mapping, Sequence, Tuple

import torch
from safetensors import safe_open

from ..parts.base import TensorInfo

_ST_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool,
}


class WeightsError(RuntimeError):
    """The checkpoint does not hold what the model needs.  ``missing``, ``unexpected`` and
    ``wrong_shape`` carry the details the message lists."""

    def __init__(self, where: str, missing: Sequence[str], unexpected: Sequence[str],
                 wrong_shape: Sequence[Tuple[str, tuple, tuple]], other: Sequence[str] = ()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.other = list(other)
        lines = [f"{where}: checkpoint does not match the model"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}):")
            lines += [f"    {n}" for n in self.missing]
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}):")
            lines += [f"    {n}" for n in self.unexpected]
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}):")
            lines += [f"    {n}: expected {tuple(e)}, found {tuple(g)}" for n, e, g in self.wrong_shape]
        lines += [f"  {o}" for o in self.other]
        super().__init__("\n".join(lines))


def shard_files(model_dir: str) -> List[str]:
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.exists(index):
        with open(index, "r", encoding="utf-8") as f:
            weight_map = json.load(f)["weight_map"]
        return sorted({os.path.join(model_dir, v) for v in weight_map.values()})
    files = sorted(glob.glob(os.path.join(model_dir, "*.safetensors")))
    if not files:
        raise FileNotFoundError(f"no .safetensors file under {model_dir}")
    return files


class Checkpoint:
    """Names, shapes and dtypes of every tensor in the folder (read from the headers only), and
    the tensors themselves on request."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        self.files = shard_files(model_dir)
        self._where: Dict[str, str] = {}
        self.shapes: Dict[str, tuple] = {}
        self.dtypes: Dict[str, torch.dtype] = {}
        for path in self.files:
            try:
                with safe_open(path, framework="pt", device="cpu") as f:
                    for name in f.keys():
                        sl = f.get_slice(name)
                        self._where[name] = path
                        self.shapes[name] = tuple(sl.get_shape())
                        self.dtypes[name] = _ST_DTYPES.get(sl.get_dtype(), None)
            except Exception as e:  # truncated or corrupt file
                raise WeightsError(model_dir, [], [], [], [f"cannot read {os.path.basename(path)}: {e}"]) from e
        self._open: Dict[str, object] = {}

    def names(self) -> List[str]:
        return sorted(self._where)

    def has(self, name: str) -> bool:
        return name in self._where

    def check(self, expected: Mapping[str, TensorInfo]) -> None:
        missing = [n for n, info in expected.items() if n not in self._where and not info.optional]
        unexpected = [n for n in self._where if n not in expected]
        wrong = [(n, info.shape, self.shapes[n]) for n, info in expected.items()
                 if n in self._where and tuple(info.shape) != self.shapes[n]]
        other = [f"{n}: dtype of the stored tensor is not supported" for n in expected
                 if n in self._where and (self.dtypes[n] is None or self.dtypes[n] == torch.bool)]
        if missing or unexpected or wrong or other:
            raise WeightsError(self.model_dir, sorted(missing), sorted(unexpected), sorted(wrong), other)

    def read(self, name: str) -> torch.Tensor:
        """The tensor as stored, on the CPU."""
        path = self._where[name]
        with safe_open(path, framework="pt", device="cpu") as f:
            return f.get_tensor(name)
