"""The command line as a user runs it (``python -m dryft_b200 ...``), in the manner of hari495/dryft's tools
(``agent/verify.py:182-190``, ``agent/bench.py:181-192``): ``random-model`` writes a folder the plain
implementation reads; ``generate`` prints exactly the plain implementation's tokens, greedy and sampled;
``bench`` prints one JSON line per workload."""

import json
import os
import subprocess
import sys

import pytest
import torch

import helpers as H
import plain_qwen3 as P

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args, timeout=600):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    return subprocess.run([sys.executable, "-m", "dryft_b200", *args], capture_output=True, text=True, cwd=ROOT, env=env,
                          timeout=timeout)


def test_random_model_writes_a_folder_the_plain_implementation_reads(tmp_path):
    out = str(tmp_path / "m")
    r = _run("random-model", "--preset", "tiny-b", "--seed", "1", "--std", "0.08", "--out", out)
    assert r.returncode == 0, r.stderr
    assert r.stdout.strip().splitlines()[-1] == out
    cfg = json.load(open(os.path.join(out, "config.json")))
    assert cfg["architectures"] == ["Qwen3ForCausalLM"] and cfg["hidden_size"] == 80 and cfg["tie_word_embeddings"] is False
    plain = P.load_plain(out, torch.float32)
    lg = plain.logits([1, 2, 3, 4, 5])
    assert lg.shape == (5, 384) and torch.isfinite(lg).all() and float(lg.std()) > 0
    # the same seed gives the same tensors; another seed gives others; --dtype float32 stores 32-bit tensors
    again = str(tmp_path / "m2")
    assert _run("random-model", "--preset", "tiny-b", "--seed", "1", "--std", "0.08", "--out", again).returncode == 0
    other = str(tmp_path / "m3")
    assert _run("random-model", "--preset", "tiny-b", "--seed", "2", "--std", "0.08", "--dtype", "float32", "--out", other).returncode == 0
    _, t1 = P.read_model_dir(out)
    _, t2 = P.read_model_dir(again)
    _, t3 = P.read_model_dir(other)
    assert set(t1) == set(t2) == set(t3) and "lm_head.weight" in t1
    assert all(torch.equal(t1[n], t2[n]) for n in t1)
    assert not torch.equal(t1["lm_head.weight"].float(), t3["lm_head.weight"].float())
    assert t1["lm_head.weight"].dtype == torch.bfloat16 and t3["lm_head.weight"].dtype == torch.float32


def test_random_model_from_a_config_file_and_unknown_names(tmp_path):
    cfg = H.config_dict("c")
    path = tmp_path / "config.json"
    path.write_text(json.dumps(cfg))
    out = str(tmp_path / "m")
    assert _run("random-model", "--config", str(path), "--seed", "3", "--out", out).returncode == 0
    got = json.load(open(os.path.join(out, "config.json")))
    assert got["sliding_window"] == 40 and got["num_hidden_layers"] == 4
    r = _run("random-model", "--preset", "no-such-shape", "--out", str(tmp_path / "x"))
    assert r.returncode != 0 and "no-such-shape" in r.stderr
    r = _run("generate", "--prompt-ids", "1,2")          # neither --model nor --tiny nor --preset
    assert r.returncode != 0 and "--model" in (r.stderr + r.stdout)


@pytest.mark.gpu
def test_generate_prints_the_plain_implementations_tokens(model_dirs):
    plain = P.load_plain(model_dirs["b"], torch.float32)
    prompts = H.prompts_for("b", [1, 7, 16, 31], seed=9)
    args = sum((["--prompt-ids", ",".join(map(str, p))] for p in prompts), [])
    r = _run("generate", "--model", model_dirs["b"], "--dtype", "float32", "--max-new-tokens", "8", *args)
    assert r.returncode == 0, r.stderr
    rows = [json.loads(ln) for ln in r.stdout.strip().splitlines()]
    assert [row["prompt_len"] for row in rows] == [1, 7, 16, 31]
    assert [row["tokens"] for row in rows] == P.plain_generate(plain, prompts, 8)
    r = _run("generate", "--model", model_dirs["b"], "--dtype", "float32", "--max-new-tokens", "8", "--temperature", "0.7",
             "--top-k", "20", "--seed", "1", *args)
    assert r.returncode == 0, r.stderr
    rows = [json.loads(ln) for ln in r.stdout.strip().splitlines()]
    assert [row["tokens"] for row in rows] == P.plain_generate(plain, prompts, 8, temperature=0.7, top_k=20, seed=1)
    # a stop token ends its sequence (the token is printed, nothing after it); the model comes from the environment
    free = P.plain_generate(plain, prompts, 8)
    stop = free[2][3]
    env_run = subprocess.run([sys.executable, "-m", "dryft_b200", "generate", "--dtype", "float32", "--max-new-tokens", "8",
                              "--stop-token-id", str(stop), *args], capture_output=True, text=True, cwd=ROOT, timeout=600,
                             env=dict(os.environ, DRYFT_MODEL_PATH=model_dirs["b"], PYTHONPATH=ROOT))
    assert env_run.returncode == 0, env_run.stderr
    rows = [json.loads(ln) for ln in env_run.stdout.strip().splitlines()]
    assert [row["tokens"] for row in rows] == P.plain_generate(plain, prompts, 8, stop_token_ids=[stop])


@pytest.mark.gpu
def test_bench_tiny_prints_one_line_per_workload():
    r = _run("bench", "--tiny", "--workload", "one,1,9,6", "--workload", "four,4,5,8", "--samples", "2")
    assert r.returncode == 0, r.stderr
    rows = [json.loads(ln) for ln in r.stdout.strip().splitlines()]
    assert [row["workload"] for row in rows] == ["one", "four"]
    for row, (b, n_out) in zip(rows, ((1, 6), (4, 8))):
        assert row["batch"] == b and row["out"] == n_out
        assert row["tok_s"] > 0 and row["ttft_ms"] > 0 and row["tpot_ms"] > 0 and row["total_ms"] >= row["ttft_ms"]
        assert 0 <= row["spread"]
    r = _run("generate", "--tiny", "--workload", "demo,3,9,4", "--temperature", "0.7", "--top-k", "20", "--seed", "1")
    assert r.returncode == 0, r.stderr
    rows = [json.loads(ln) for ln in r.stdout.strip().splitlines()]
    assert len(rows) == 3 and all(row["prompt_len"] == 9 and len(row["tokens"]) == 4 for row in rows)
