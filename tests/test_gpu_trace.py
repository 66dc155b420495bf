"""``bin/trace_run`` as a user runs it: a child process fed JSON steps on standard input.  The same
requests are replayed whole, with the last 32 tokens one by one, and in batches of unequal lengths
(fewer tokens of cache than all requests together, so slots and pages are used again), in 32-bit and
in bfloat16, and every logit row is compared with the plain implementation."""

import os

import numpy as np
import pytest
import torch

import helpers as H
import plain_qwen3 as P

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
_T = {"float32": torch.float32, "bfloat16": torch.bfloat16}
_plains = {}


def plain(model_dirs, name, dtype):
    key = (name, dtype)
    if key not in _plains:
        _plains[key] = P.load_plain(model_dirs[name], dtype)
    return _plains[key]


def compare(got: np.ndarray, name, tokens, rows, model_dirs, dtype, what):
    got = torch.from_numpy(np.ascontiguousarray(got))
    p32 = plain(model_dirs, name, torch.float32).logits(tokens)[rows]
    assert torch.isfinite(got).all(), what
    if dtype == "float32":
        e = H.rel_err(got, p32)
        assert e <= H.FP32_TOL, f"{what}: off by {e:.3g}"
    else:
        pb = plain(model_dirs, name, torch.bfloat16).logits(tokens)[rows]
        tol = H.bf16_tol(pb, p32)
        e = H.rel_err(got, pb)
        assert e <= tol, f"{what}: off by {e:.3g} (allowed {tol:.3g})"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["a", "b", "c", "d"])
def test_trace_replay_every_way_of_cutting(model_dirs, tmp_path, name, dtype):
    lengths = [40, 97, 33, 150, 64, 71]
    reqs = [H.prompts_for(name, [n], seed=200 + i)[0] for i, n in enumerate(lengths)]
    # room for about half of the requests at a time: slots and pages must be given back and reused
    tr = H.TraceRun(model_dirs[name], dtype, str(tmp_path / "out"), max_tokens=320)
    try:
        # 1. each request alone and whole, logits at every place
        for i, toks in enumerate(reqs):
            got = tr.step([{"id": f"w{i}", "tokens": toks, "want": list(range(len(toks)))}], end=[f"w{i}"])
            compare(got, name, toks, list(range(len(toks))), model_dirs, dtype, f"{name} whole request {i}")
        # 2. the last 32 tokens one by one
        for i, toks in enumerate(reqs):
            n = len(toks)
            head = n - 32
            rows = [tr.step([{"id": f"d{i}", "tokens": toks[:head], "want": [head - 1]}])]
            for t in range(head, n):
                rows.append(tr.step([{"id": f"d{i}", "tokens": [toks[t]], "want": [0]}], end=[f"d{i}"] if t == n - 1 else []))
            compare(np.concatenate(rows), name, toks, list(range(head - 1, n)), model_dirs, dtype,
                    f"{name} request {i} last 32 one by one")
        # 3. batches of unequal lengths: prompts together, then one token each, shorter ones end earlier
        for bi, members in enumerate([[0, 2, 4], [1, 5], [3, 2]]):
            prompt_len = {i: max(1, len(reqs[i]) - 20 - 7 * k) for k, i in enumerate(members)}
            got = {i: [] for i in members}
            rows_of = {i: [] for i in members}
            out = tr.step([{"id": f"b{bi}_{i}", "tokens": reqs[i][:prompt_len[i]], "want": [prompt_len[i] - 1]} for i in members])
            for j, i in enumerate(members):
                got[i].append(out[j:j + 1])
                rows_of[i].append(prompt_len[i] - 1)
            fed = dict(prompt_len)
            alive = list(members)
            while alive:
                ending = [i for i in alive if fed[i] + 1 >= len(reqs[i])]
                out = tr.step([{"id": f"b{bi}_{i}", "tokens": [reqs[i][fed[i]]], "want": [0]} for i in alive],
                              end=[f"b{bi}_{i}" for i in ending])
                for j, i in enumerate(alive):
                    got[i].append(out[j:j + 1])
                    rows_of[i].append(fed[i])
                    fed[i] += 1
                alive = [i for i in alive if i not in ending]
            for i in members:
                compare(np.concatenate(got[i]), name, reqs[i], rows_of[i], model_dirs, dtype, f"{name} batch {bi} request {i}")
        # a step in which nothing is wanted writes no file
        n_before = len(os.listdir(tr.out_dir))
        assert tr.step([{"id": "q", "tokens": reqs[0][:5], "want": []}], end=["q"]) is None
        assert len(os.listdir(tr.out_dir)) == n_before
    finally:
        assert tr.close() == 0
