"""Command line, in the manner of hari495/dryft's tools (``agent/verify.py:182-190``,
``agent/bench.py:181-192``): ``--model`` (default ``$DRYFT_MODEL_PATH``), ``--tiny`` for a random tiny
model, ``--seed``, ``--samples``, ``--workload name,b,in,out``.  Token ids in and out, no tokenizer
(as there, ``AGENTS.md:120``).

    python -m dryft_b200 generate --model DIR --prompt-ids 1,2,3 --prompt-ids 4,5 --max-new-tokens 8
    python -m dryft_b200 generate --tiny --workload demo,3,9,8 --temperature 0.7 --top-k 20 --seed 1
    python -m dryft_b200 bench --model DIR --workload b1,1,512,32 --workload b16,16,512,128 --samples 5
    python -m dryft_b200 random-model --preset tiny-b --seed 1 --out DIR
    python -m dryft_b200 replay --model DIR --dtype float32 --out DIR --max-tokens 4096 < trace.jsonl
"""

from __future__ import annotations

import argparse
import json
import os
import random
import statistics
import sys
import tempfile
import time
from typing import List


def _workload(text: str):
    name, b, inp, out = text.split(",")
    return name, int(b), int(inp), int(out)


def _model_dir(args) -> str:
    if args.tiny:
        from .config import preset
        from .weights import write_random_model

        d = os.path.join(tempfile.gettempdir(), f"dryft-b200-tiny-{os.getuid()}")
        if not os.path.isfile(os.path.join(d, "model.safetensors")):
            write_random_model(preset("tiny-a"), 0, d, std=0.08)
        return d
    if not args.model:
        raise SystemExit("give --model DIR (or set DRYFT_MODEL_PATH), --preset NAME, or --tiny")
    return args.model


def _engine(args):
    from .engine.api import Engine

    kw = dict(dtype=args.dtype, cuda_graphs=not args.no_cuda_graph)
    if args.max_batch:
        kw["max_batch"] = args.max_batch
    if args.max_seq_len:
        kw["max_seq_len"] = args.max_seq_len
    if args.tiny:
        kw.setdefault("max_batch", 8)
        kw.setdefault("max_seq_len", 128)
    if getattr(args, "preset", None) and not args.tiny and not args.model:
        # random weights of a named shape, made on the device (no folder is written)
        from .config import preset

        return Engine.from_config(preset(args.preset), seed=args.weights_seed, **kw)
    return Engine(_model_dir(args), **kw)


def cmd_generate(args) -> int:
    eng = _engine(args)
    prompts: List[List[int]] = [[int(t) for t in p.split(",") if t] for p in args.prompt_ids]
    rng = random.Random(args.seed)
    for w in args.workload:
        _, b, inp, _ = _workload(w)
        prompts += [[rng.randrange(eng.config.vocab_size) for _ in range(inp)] for _ in range(b)]
    if not prompts:
        raise SystemExit("nothing to generate from: give --prompt-ids or --workload")
    if args.max_new_tokens is not None:
        n = args.max_new_tokens
    else:
        n = max((_workload(w)[3] for w in args.workload), default=16)   # a workload names its own output length
    out = eng.generate_many(prompts, n, temperature=args.temperature, top_k=args.top_k, seed=args.seed,
                            stop_token_ids=args.stop_token_id)
    for p, o in zip(prompts, out):
        print(json.dumps({"prompt_len": len(p), "tokens": o}))
    return 0


def cmd_bench(args) -> int:
    """Median tok/s (batch x output tokens / total seconds, prefill included), TTFT and TPOT per
    workload, as ``agent/bench.py:96-126`` measures them."""
    import torch

    eng = _engine(args)
    rng = random.Random(args.seed)
    for w in args.workload or ["b1,1,512,32"]:
        name, b, inp, out = _workload(w)
        totals, ttfts = [], []
        for s in range(args.samples + 1):  # the first sample is the warm-up
            ids = [[rng.randrange(eng.config.vocab_size) for _ in range(inp)] for _ in range(b)]
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            ttft = None
            for _ in eng.generate(ids, out):
                if ttft is None:
                    ttft = time.perf_counter() - t0
            torch.cuda.synchronize()
            if s:
                totals.append(time.perf_counter() - t0)
                ttfts.append(ttft)
        total, ttft = statistics.median(totals), statistics.median(ttfts)
        print(json.dumps({"workload": name, "batch": b, "in": inp, "out": out, "tok_s": b * out / total,
                          "total_ms": total * 1e3, "ttft_ms": ttft * 1e3,
                          "tpot_ms": (total - ttft) / max(1, out - 1) * 1e3,
                          "spread": (max(totals) - min(totals)) / total}))
    return 0


def cmd_random_model(args) -> int:
    import torch

    from .config import preset
    from .weights import write_random_model

    cfg = preset(args.preset) if args.preset else json.load(open(args.config))
    dt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[args.dtype]
    print(write_random_model(cfg, args.seed, args.out, dtype=dt, std=args.std))
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="dryft_b200")
    sub = ap.add_subparsers(dest="cmd", required=True)

    def common(p):
        p.add_argument("--model", default=os.environ.get("DRYFT_MODEL_PATH"))
        p.add_argument("--tiny", action="store_true", help="a random tiny Qwen3 instead of --model")
        p.add_argument("--preset", default=None, help="random weights of a named shape instead of --model (tiny-a, tiny-b, qwen3-4b, ...)")
        p.add_argument("--weights-seed", type=int, default=0, help="seed of --preset's weights")
        p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
        p.add_argument("--seed", type=int, default=0)
        p.add_argument("--workload", action="append", default=[], help="name,b,in,out")
        p.add_argument("--max-batch", type=int, default=0)
        p.add_argument("--max-seq-len", type=int, default=0)
        p.add_argument("--no-cuda-graph", action="store_true")

    g = sub.add_parser("generate", help="generate token ids from token ids")
    common(g)
    g.add_argument("--prompt-ids", action="append", default=[], help="comma-separated token ids; may repeat")
    g.add_argument("--max-new-tokens", type=int, default=None, help="default: the workloads' output length, else 16")
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--top-k", type=int, default=0)
    g.add_argument("--stop-token-id", type=int, action="append", default=[])
    g.set_defaults(fn=cmd_generate)

    b = sub.add_parser("bench", help="time workloads through Engine.generate")
    common(b)
    b.add_argument("--samples", type=int, default=5)
    b.set_defaults(fn=cmd_bench)

    t = sub.add_parser("replay", help="feed a token trace step by step and write logits (bin/trace_run)", add_help=False)
    t.set_defaults(fn=None)

    r = sub.add_parser("random-model", help="write a model folder with random weights")
    r.add_argument("--preset", default=None)
    r.add_argument("--config", default=None, help="a config.json to take the sizes from")
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--std", type=float, default=0.02)
    r.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    r.add_argument("--out", required=True)
    r.set_defaults(fn=cmd_random_model)

    argv = list(sys.argv[1:] if argv is None else argv)
    if argv[:1] == ["replay"]:   # the replay program parses its own options (those of bin/trace_run)
        from .replay import main as replay_main

        return replay_main(argv[1:])
    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
