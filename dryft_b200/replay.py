"""Trace replay: feed given token ids through a model step by step and write logits
(``bin/trace_run`` and ``python -m dryft_b200 replay`` both run ``main`` below).

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Reads one JSON object per line from standard input:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries``: for each request its next tokens and the places among them whose logits are wanted.
``end``: requests that are finished after this step; their slot and pages are given back.
For a step in which something is wanted, ``<out>/<step>.f32`` receives the logits at the wanted
places, in the order of the entries and of ``want``, as little-endian float32 ``[wanted, vocab]``.
After every step a line ``done <step>`` is printed and flushed.  Nothing is sampled.

It drives the library's own model, step function, cache and kernels — the ones generation uses —
and has no forward pass, cache or loader of its own.  In spirit it is the teacher-forced replay of
hari495/dryft's ``agent/verify.py:100-109``, run through the engine itself instead of an oracle.
"""

from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="replay a token trace through dryft_b200 and dump logits")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to a multiple of 64)")
    args = ap.parse_args(argv)

    import numpy as np
    import torch

    from .engine.api import Engine, EngineOptions
    from .ops import kernels

    page = EngineOptions().page_size   # requests are counted in the cache's own unit
    n_tokens = max(page, (args.max_tokens + page - 1) // page * page)
    opts = EngineOptions(dtype=args.dtype, max_batch=min(n_tokens // page, 4096), max_seq_len=n_tokens,
                         max_tokens=n_tokens, page_size=page, cuda_graphs=False)
    engine = Engine(args.model, opts)
    os.makedirs(args.out, exist_ok=True)
    slot_of = {}

    with torch.cuda.device(engine.device), torch.inference_mode():
        for line in sys.stdin:
            line = line.strip()
            if not line:
                continue
            rec = json.loads(line)
            step = rec["step"]
            entries = rec.get("entries", [])
            new_ids = [e["id"] for e in entries if e["id"] not in slot_of]
            if len(set(new_ids)) != len(new_ids):
                raise ValueError(f"step {step}: a request id occurs twice")
            for rid, slot in zip(new_ids, engine.cache.open_sequences(len(new_ids))):
                slot_of[rid] = slot
            if entries:
                logits = engine.stepper.step([slot_of[e["id"]] for e in entries], [e["tokens"] for e in entries],
                                             [e.get("want", []) for e in entries])
                if logits is not None:
                    arr = logits.to(torch.float32).cpu().numpy().astype("<f4", copy=False)
                    tmp = os.path.join(args.out, f".{step}.f32.tmp")
                    arr.tofile(tmp)
                    os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
            ended = [rid for rid in rec.get("end", [])]
            unknown = [rid for rid in ended if rid not in slot_of]
            if unknown:
                raise ValueError(f"step {step}: 'end' names requests that are not live: {unknown}")
            engine.cache.close_sequences([slot_of.pop(rid) for rid in ended])
            torch.cuda.synchronize()
            kernels.check_error_flags()
            print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
