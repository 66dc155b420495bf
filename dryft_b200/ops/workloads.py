"""Whole workloads of the larger shapes through ``Engine.generate`` (host tokens in and out), random weights:

    python -m dryft_b200.ops.workloads 8b        Qwen3-8B shape, 16 prompts of 64..2,048 tokens, 256 greedy steps
    python -m dryft_b200.ops.workloads 32b-64    Qwen3-32B shape, 64 prompts of 1,024 tokens, 128 steps
    python -m dryft_b200.ops.workloads 32b-1     Qwen3-32B shape, one prompt of 16,384 tokens, 128 steps

Prints one JSON line: the time to the first token (the whole prompts in one step), then the decode steps.
hari495/dryft measures its workloads the same way, through its engine's generate (``agent/bench.py:96-126``).
"""

from __future__ import annotations

import json
import random
import sys
import time
from typing import List

import torch

from ..config import config_from_dict, preset
from ..engine.api import Engine

WORKLOADS = ("8b", "32b-64", "32b-1")


def run(name: str, prompts: List[List[int]], new: int, max_seq_len: int) -> dict:
    cfg = config_from_dict(preset(name))
    batch = len(prompts)
    eng = Engine.from_config(cfg, seed=0, dtype="bfloat16", max_batch=batch, max_seq_len=max_seq_len,
                             max_tokens=sum(((len(p) + new + 63) // 64 + 1) * 64 for p in prompts))
    first = t0 = t1 = 0.0
    steps = 0
    for _ in range(3):   # the third pass is the measurement (libraries loaded by the first, the prompt step's graph captured by the second)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        steps = 0
        for _tokens in eng.generate(prompts, new):
            if steps == 0:
                torch.cuda.synchronize()
                first = time.perf_counter()
            steps += 1
        torch.cuda.synchronize()
        t1 = time.perf_counter()
    prompt_tokens = sum(len(p) for p in prompts)
    return {"shape": name, "batch": batch, "prompt_tokens": prompt_tokens, "new": new,
            "prefill_ms": round((first - t0) * 1e3, 1), "prefill_tok_s": round(prompt_tokens / (first - t0)),
            "decode_ms_per_step": round((t1 - first) * 1e3 / (steps - 1), 3),
            "decode_tok_s": round(batch * (steps - 1) / (t1 - first))}


def main(argv) -> int:
    if len(argv) != 2 or argv[1] not in WORKLOADS:
        print("usage: python -m dryft_b200.ops.workloads " + "|".join(WORKLOADS), file=sys.stderr)
        return 2
    rng = random.Random(0)
    vocab = config_from_dict(preset("qwen3-8b")).vocab_size
    if argv[1] == "8b":
        lengths = [rng.randint(64, 2048) for _ in range(16)]
        out = run("qwen3-8b", [[rng.randrange(vocab) for _ in range(n)] for n in lengths], 256, 2048 + 256 + 64)
    elif argv[1] == "32b-64":
        out = run("qwen3-32b", [[rng.randrange(vocab) for _ in range(1024)] for _ in range(64)], 128, 1024 + 128 + 64)
    else:
        out = run("qwen3-32b", [[rng.randrange(vocab) for _ in range(16384)]], 128, 16384 + 128 + 64)
    print(json.dumps(out), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv))
