"""Shared test helpers: the tiny configurations, model folders, prompts, error measures and a driver
for ``bin/trace_run``.  Nothing here imports the product's model code except through the public
entry points the tests exercise."""

from __future__ import annotations

import json
import os
import subprocess
import sys
from typing import Dict, List, Sequence

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Three tiny configurations of the one architecture, differing in every size and option:
# layers, width (powers of two and not), head counts, group size (2 / 2 / 3), head size (16 / 32 / 48),
# q width equal to the hidden width or not, intermediate size, vocabulary (256 / 384 / 331, a prime),
# rope theta, eps, tied or untied head, maximum position, and a sliding window on some layers.
TINY: Dict[str, dict] = {
    "a": dict(num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
              intermediate_size=128, vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6,
              tie_word_embeddings=True, max_position_embeddings=512),
    "b": dict(num_hidden_layers=3, hidden_size=80, num_attention_heads=6, num_key_value_heads=3, head_dim=32,
              intermediate_size=224, vocab_size=384, rope_theta=1000000.0, rms_norm_eps=1e-5,
              tie_word_embeddings=False, max_position_embeddings=1024),
    "c": dict(num_hidden_layers=4, hidden_size=96, num_attention_heads=6, num_key_value_heads=2, head_dim=48,
              intermediate_size=176, vocab_size=331, rope_theta=500000.0, rms_norm_eps=3e-6,
              tie_word_embeddings=False, max_position_embeddings=2048,
              use_sliding_window=True, sliding_window=40, max_window_layers=1),
    # widths that are multiples of 256: the decode products compiled per inner size and the norm split
    # over two launches only run at such widths (hidden 256, q width 512, intermediate 512)
    "d": dict(num_hidden_layers=3, hidden_size=256, num_attention_heads=8, num_key_value_heads=2, head_dim=64,
              intermediate_size=512, vocab_size=300, rope_theta=10000.0, rms_norm_eps=1e-6,
              tie_word_embeddings=False, max_position_embeddings=512),
}
SEEDS = {"a": 0, "b": 1, "c": 2, "d": 3}
# normal(0, 0.02) weights give nearly flat logits on models this small; a wider spread makes every
# stage matter (the reference multiplies its tiny model's weights by 4, agent/verify.py:49-51)
STD = 0.08


def config_dict(name: str) -> dict:
    base = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_act": "silu",
            "attention_bias": False, "rope_scaling": None}
    base.update(TINY[name])
    return base


def make_model_dir(name: str, out_dir: str, dtype: torch.dtype = torch.bfloat16, std: float = STD) -> str:
    from dryft_b200.weights import write_random_model

    return write_random_model(config_dict(name), SEEDS[name], out_dir, dtype=dtype, std=std)


def prompts_for(name: str, lengths: Sequence[int], seed: int = 0) -> List[List[int]]:
    g = torch.Generator().manual_seed(1000 + seed)
    vocab = TINY[name]["vocab_size"]
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]


def rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    """max |a - b| / max |b|."""
    a = a.detach().to(torch.float64).cpu()
    b = b.detach().to(torch.float64).cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


# 32-bit path: sums in another order, 2-ulp device functions (sincosf, expf, rsqrtf)
FP32_TOL = 2e-5


def bf16_tol(plain_bf16: torch.Tensor, plain_fp32: torch.Tensor) -> float:
    """What bfloat16 rounding alone does to these logits (plain bf16 vs plain fp32 on the same
    weights), doubled: an engine result may round differently at every stage, so it may sit as far
    from the plain bf16 result as that one sits from the exact one, but a wrong key, position or slot
    moves logits by far more."""
    return 2.0 * rel_err(plain_bf16, plain_fp32) + 1e-3


# --------------------------------------------------------------------------- bin/trace_run driver
class TraceRun:
    """Runs ``bin/trace_run`` as a child process and feeds it steps one at a time."""

    def __init__(self, model_dir: str, dtype: str, out_dir: str, max_tokens: int):
        self.out_dir = out_dir
        self.vocab = json.load(open(os.path.join(model_dir, "config.json")))["vocab_size"]
        cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
               "--out", out_dir, "--max-tokens", str(max_tokens)]
        self.proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
        self.n = 0

    def step(self, entries: List[dict], end: Sequence[str] = ()) -> "np.ndarray | None":
        step = self.n
        self.n += 1
        self.proc.stdin.write(json.dumps({"step": step, "entries": entries, "end": list(end)}) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline().strip()
        if line != f"done {step}":
            rc = self.proc.poll()
            raise RuntimeError(f"trace_run answered {line!r} to step {step} (exit code {rc})")
        wanted = sum(len(e.get("want", [])) for e in entries)
        if wanted == 0:
            return None
        arr = np.fromfile(os.path.join(self.out_dir, f"{step}.f32"), dtype="<f4")
        return arr.reshape(wanted, self.vocab)

    def close(self) -> int:
        self.proc.stdin.close()
        rc = self.proc.wait(timeout=120)
        return rc
