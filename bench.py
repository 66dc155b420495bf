"""Benchmark of the flagship serving step: decode tokens a second of a Qwen3-4B-shaped model.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one decode step of the whole batch.  The default run has the layer sizes of the
Qwen3-4B shape (36 layers, hidden 2560, 32/8 heads of 128, intermediate 9728, vocabulary 151936, tied
head) with random weights, a batch of 8 sequences with 512-token prompts, and times K decode steps
(device time, CUDA events, after W warm-up steps).  One JSON line is printed:

  value     decoded tokens a second (batch * K / device time of the K steps; tokens stay on the device)
  e2e       the same through the Python entry point ``Engine.generate``: host token lists in, one host
            list out per step (every step copies its slot list host->device from pinned memory and
            reads the chosen tokens device->host)
  prefill   one 2,048-token prompt through the step function: tokens a second, ms, and the step's
            flops / time / the bf16 peak of a product timed alone (the step is timed alone too)
  spread, peak_mem_gib   (slowest - fastest) / median over the eighths of the timed region; the allocator's peaks
  roofline  the decode step against HBM: bytes it has to read (every weight once, and the cache of
            the live requests) / its time, against the measured copy bandwidth
  points    decode tokens a second at batch 1 and 64
  clocks    SM clock under load, sampled with nvidia-smi during the timed region

The method follows hari495/dryft's ``agent/bench.py:96-126`` (warm-up, synchronize on both sides,
seeded uniform token ids, ``bench.py:111-119``); its achieved-bandwidth figure (``bench.py:171-172``) is
the ``roofline`` entry.

``--impl reference`` times hari495/dryft itself for the same metric: its unmodified ``engine/`` folder
(kept under ``baseline/_ref/engine``; the project has no setup.py or pyproject.toml, so it is a plain copy
rather than a pip install) is put on ``sys.path`` and driven through its own public entry point,
``Engine(model_path).generate(input_ids, max_new_tokens)`` (``engine/engine.py:28-30,138-166``), on a
Qwen3-4B-shaped random-weights folder written to a temporary directory.  Nothing of ``dryft_b200`` is
imported on that path.
"""

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0      # earlier measurement on this pool, used only if MEASURED_PEAKS.json is absent
FALLBACK_BF16_TFLOPS = 1590.0


def peaks():
    """(copy bandwidth GB/s, bf16 TFLOP/s of a product timed alone, source).  The prefill step is timed alone between
    synchronisations, so its fraction is taken against the burst figure, not the one sustained under the power cap."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            p = json.load(open(path))
            return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, "fallback"


class ClockSampler:
    """nvidia-smi clock samples while the timed region runs (read-only queries)."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in self.rows if len(r) >= 6 for i in range(4) if r[2 + i].lower().startswith("active")})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def random_prompts(batch, length, vocab, seed):
    import random

    rng = random.Random(seed)
    return [[rng.randrange(vocab) for _ in range(length)] for _ in range(batch)]


def decode_device_time(eng, batch, prompt_len, steps, warmup, seed):
    """K decode steps of one batch, tokens never leaving the device: ms per step (CUDA events)."""
    import torch

    from dryft_b200.ops import kernels as K
    from dryft_b200.sampling.sampler import SamplingParams, choose

    prompts = random_prompts(batch, prompt_len, eng.config.vocab_size, seed)
    params = SamplingParams()
    with torch.inference_mode():
        slots = eng.cache.open_sequences(batch)
        try:
            logits = eng.stepper.step(slots, prompts, [[prompt_len - 1]] * batch)
            row_slot = torch.tensor(slots, dtype=torch.int32, device=eng.device)
            choose(logits, params, row_slot=row_slot, last_token=eng.cache.last_token)

            def one():
                lg = eng.stepper.decode_from_state(slots)
                choose(lg, params, row_slot=eng.stepper.last_decode_slots, last_token=eng.cache.last_token)

            for _ in range(warmup):
                one()
            torch.cuda.synchronize()
            n0 = K.launch_count
            ctx0 = eng.cache.len_host[slots[0]]
            # one event every `every` steps: the whole region gives the time, the pieces give its spread
            every = max(1, steps // 8)
            marks = [torch.cuda.Event(enable_timing=True)]
            marks[0].record()
            for i in range(steps):
                one()
                if (i + 1) % every == 0 or i + 1 == steps:
                    marks.append(torch.cuda.Event(enable_timing=True))
                    marks[-1].record()
            torch.cuda.synchronize()
            ms = marks[0].elapsed_time(marks[-1]) / steps
            pieces = [a.elapsed_time(b) / every for a, b in zip(marks[:-1], marks[1:])][: steps // every]
            spread = (max(pieces) - min(pieces)) / statistics.median(pieces) if len(pieces) > 1 else 0.0
            launches = K.launch_count - n0
            ctx1 = eng.cache.len_host[slots[0]]
        finally:
            eng.cache.close_sequences(slots)
    decode_device_time.spread = spread
    return ms, launches, (ctx0 + ctx1) / 2.0


def decode_e2e(eng, batch, prompt_len, steps, seed):
    """The same through Engine.generate: host lists in, a host list out per step."""
    import torch

    prompts = random_prompts(batch, prompt_len, eng.config.vocab_size, seed)
    be = eng._backend
    for _ in eng.generate(prompts, 4):  # warm-up of this batch shape
        pass
    torch.cuda.synchronize()
    h0, d0 = be.h2d_bytes, be.d2h_bytes
    t_first = None
    n = 0
    for out in eng.generate(prompts, steps + 1):
        if t_first is None:
            torch.cuda.synchronize()
            t_first = time.perf_counter()
            h1, d1 = be.h2d_bytes, be.d2h_bytes
        n += 1
    torch.cuda.synchronize()
    dt = time.perf_counter() - t_first
    assert n == steps + 1
    return batch * steps / dt, (be.h2d_bytes - h1) // steps, (be.d2h_bytes - d1) // steps


def prefill_time(eng, tokens, iters, seed):
    import torch

    prompt = random_prompts(1, tokens, eng.config.vocab_size, seed)[0]
    times = []
    with torch.inference_mode():
        for i in range(iters + 2):
            (slot,) = eng.cache.open_sequences(1)
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            eng.stepper.step([slot], [prompt], [[tokens - 1]])
            e.record()
            torch.cuda.synchronize()
            eng.cache.close_sequences([slot])
            if i >= 2:
                times.append(s.elapsed_time(e))
    return statistics.median(times)


# ----------------------------------------------------------------------------- the reference arm
REF_ENGINE_DIR = os.path.join(ROOT, "baseline", "_ref", "engine")

# the checkpoint facts hari495/dryft pins (engine/dryft_qwen3/config.py:53-70): the benchmark shape
REF_CONFIG = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 36, "hidden_size": 2560,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 9728,
    "hidden_act": "silu", "vocab_size": 151936, "tie_word_embeddings": True, "rms_norm_eps": 1e-6,
    "rope_theta": 5000000, "rope_scaling": None, "max_position_embeddings": 262144, "attention_bias": False,
    "torch_dtype": "bfloat16",
}


def write_reference_model(out_dir, seed):
    """config.json + model.safetensors of the benchmark shape: normal(0, 0.02) matrices, norm weights
    1 + normal(0, 0.02), bfloat16, tied head (no lm_head.weight).  Drawn on the GPU (4 G values), saved once."""
    import torch
    from safetensors.torch import save_file

    c = REF_CONFIG
    H, D, I, V = c["hidden_size"], c["head_dim"], c["intermediate_size"], c["vocab_size"]
    Hq, Hkv = c["num_attention_heads"] * D, c["num_key_value_heads"] * D
    gen = torch.Generator(device="cuda").manual_seed(seed)

    def mat(*shape):
        return (torch.randn(shape, generator=gen, device="cuda", dtype=torch.float32) * 0.02).to(torch.bfloat16).cpu()

    def vec(n):
        return (1.0 + torch.randn((n,), generator=gen, device="cuda", dtype=torch.float32) * 0.02).to(torch.bfloat16).cpu()

    t = {"model.embed_tokens.weight": mat(V, H), "model.norm.weight": vec(H)}
    for i in range(c["num_hidden_layers"]):
        p = f"model.layers.{i}."
        t[p + "input_layernorm.weight"] = vec(H)
        t[p + "self_attn.q_proj.weight"] = mat(Hq, H)
        t[p + "self_attn.k_proj.weight"] = mat(Hkv, H)
        t[p + "self_attn.v_proj.weight"] = mat(Hkv, H)
        t[p + "self_attn.q_norm.weight"] = vec(D)
        t[p + "self_attn.k_norm.weight"] = vec(D)
        t[p + "self_attn.o_proj.weight"] = mat(H, Hq)
        t[p + "post_attention_layernorm.weight"] = vec(H)
        t[p + "mlp.gate_proj.weight"] = mat(I, H)
        t[p + "mlp.up_proj.weight"] = mat(I, H)
        t[p + "mlp.down_proj.weight"] = mat(H, I)
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(c, f, indent=1)
    save_file(t, os.path.join(out_dir, "model.safetensors"), metadata={"format": "pt"})


def reference_arm(args) -> int:
    """hari495/dryft's own engine on the same metric and shape (batch 8, 512-token prompts, K decode steps).
    ``value`` = batch x K / the time between the first and the last yield of ``generate(ids, K + 1)``:
    host token lists in, a host list out per step, so it is an end-to-end number and ``e2e`` repeats it."""
    import shutil
    import tempfile

    def unavailable(why):
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0

    if not os.path.isfile(os.path.join(REF_ENGINE_DIR, "engine.py")):
        return unavailable("baseline/_ref/engine/engine.py is absent (hari495/dryft has no setup.py or pyproject.toml to "
                           "pip-install; its engine/ folder is copied there by hand)")
    if args.gpus != 1:
        return unavailable("hari495/dryft is a single-GPU engine (no torch.distributed call site)")
    try:
        import torch
        if not torch.cuda.is_available():
            return unavailable("no CUDA device")
        import triton  # noqa: F401  (the reference imports it directly)
    except Exception as e:  # noqa: BLE001
        return unavailable(f"import failed: {e!r}")
    warmup = max(3, args.warmup)
    batch, prompt_len, steps = args.batch, args.prompt_len, args.steps
    tmp = tempfile.mkdtemp(prefix="dryft-ref-model-")
    try:
        t0 = time.time()
        write_reference_model(tmp, args.seed)
        print(f"[bench] reference: wrote the random-weights folder in {time.time() - t0:.0f}s", file=sys.stderr, flush=True)
        sys.path.insert(0, REF_ENGINE_DIR)
        try:
            from engine import Engine as RefEngine  # baseline/_ref/engine/engine.py
            eng = RefEngine(tmp)
        except Exception as e:  # noqa: BLE001
            return unavailable(f"hari495/dryft's Engine(model_path) failed here: {e!r}"[:400])
        kernels = {n: getattr(eng.model, a, None) is not None for n, a in
                   (("rmsnorm", "_k_rms"), ("rope_qknorm", "_k_rope"), ("attn_decode", "_k_attn"), ("silu_mul", "_k_silu"))}
        prompts = random_prompts(batch, prompt_len, REF_CONFIG["vocab_size"], args.seed)
        for _ in eng.generate(prompts, warmup + 1):
            pass
        torch.cuda.synchronize()
        clocks = ClockSampler()
        clocks.start()
        t_first, n = None, 0
        for out in eng.generate(prompts, steps + 1):
            if t_first is None:
                torch.cuda.synchronize()
                t_first = time.perf_counter()
            n += 1
        torch.cuda.synchronize()
        dt = time.perf_counter() - t_first
        clock_info = clocks.stop()
        assert n == steps + 1 and len(out) == batch
        value = batch * steps / dt
        T = 2048
        long_prompt = random_prompts(1, T, REF_CONFIG["vocab_size"], args.seed + 2)
        pf = []
        for i in range(5):
            torch.cuda.synchronize()
            t1 = time.perf_counter()
            for _ in eng.generate(long_prompt, 1):
                pass
            torch.cuda.synchronize()
            if i >= 2:
                pf.append((time.perf_counter() - t1) * 1e3)
        pf_ms = statistics.median(pf)
        line = {
            "metric": "decode tok/s @ batch 8; Qwen3-4B shape BF16 (points: batch 1/64; prefill tok/s @ 2048 tok)",
            "value": value, "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": dt / steps * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic: seeded uniform token ids, random normal(0,0.02) weights", "impl": "reference",
            "config": {"model": "qwen3-4b", "layers": 36, "layers_of_shape": 36, "hidden": 2560, "q_heads": 32, "kv_heads": 8,
                       "head_dim": 128, "intermediate": 9728, "vocab": 151936, "tied_head": True, "global_batch": batch,
                       "seq_len": prompt_len, "parallelism": "single-gpu", "cuda_graphs": eng.graphs is not None,
                       "timing": "host clock between the first and last yield of Engine.generate, synchronized",
                       "triton_kernels_on": ",".join(k for k, v in kernels.items() if v) or "none (torch path)",
                       "speculation": bool(getattr(eng, "spec_ok", False))},
            # the reference's loop copies its int64 next tokens to a pinned ring every step; its inputs stay on the device
            "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 8 * batch},
            "prefill": {"value": T / (pf_ms * 1e-3), "tokens": T, "ms": pf_ms},
            "clocks": clock_info,
        }
        print(json.dumps(line))
        return 0
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the shape has (named in config)")
    ap.add_argument("--preset", default="qwen3-4b")
    ap.add_argument("--no-points", action="store_true")
    ap.add_argument("--phase", default="all", choices=["all", "decode", "prefill"],
                    help="time only one phase (for profiling); the JSON line then carries only that phase")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--small-m-max", type=int, default=None,
                    help="rows up to which decode products stream weights themselves (the engine's default if not given)")
    ap.add_argument("--engine-opt", action="append", default=[], metavar="NAME=VALUE",
                    help="an EngineOptions switch for an A/B run, e.g. norm_ahead=0, pdl=0, fuse_decode=0 (named in config)")
    args = ap.parse_args()

    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not measured")
        return 2
    warmup = max(3, args.warmup)

    import torch

    from dryft_b200.config import config_from_dict, preset
    from dryft_b200.engine.api import Engine

    raw = preset(args.preset)
    full_layers = raw["num_hidden_layers"]
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    cfg = config_from_dict(raw)
    hbm_gbs, bf16_tflops, peak_src = peaks()
    # the full run also measures batch 64; a single phase holds only what its batch needs (long contexts fit)
    max_batch = max(64, args.batch) if args.phase == "all" else args.batch
    ctx_cap = args.prompt_len + args.steps + warmup + 64
    engine_opts = {}
    for item in args.engine_opt:
        name, _, val = item.partition("=")
        engine_opts[name] = {"0": False, "1": True}.get(val, int(val) if val.lstrip("-").isdigit() else val)
    eng = Engine.from_config(cfg, seed=args.seed, dtype="bfloat16", max_batch=max_batch,
                             max_seq_len=max(raw["max_position_embeddings"], 2048 + 64, ctx_cap),
                             max_tokens=max(max_batch * (ctx_cap + 64), 4096),
                             **({"small_m_max": args.small_m_max} if args.small_m_max is not None else {}), **engine_opts)
    torch.cuda.synchronize()

    if args.phase == "prefill":
        pf_ms = prefill_time(eng, 2048, 3, args.seed + 2)
        print(json.dumps({"phase": "prefill", "tokens": 2048, "ms": pf_ms, "tok_s": 2048 / (pf_ms * 1e-3)}))
        return 0
    if args.phase == "decode":
        ms, launches, mean_ctx = decode_device_time(eng, args.batch, args.prompt_len, args.steps, warmup, args.seed)
        print(json.dumps({"phase": "decode", "batch": args.batch, "ms_per_step": ms, "tok_s": args.batch * 1000.0 / ms,
                          "launches": launches, "mean_context": mean_ctx}))
        return 0

    # the prompt step first: it is timed alone and compared with the burst peak of a product timed alone
    # (after seconds of decode steps under the power cap the same step takes up to a tenth longer)
    T = 2048
    pf_ms = prefill_time(eng, T, 5, args.seed + 2)

    clocks = ClockSampler()
    clocks.start()
    ms, launches, mean_ctx = decode_device_time(eng, args.batch, args.prompt_len, args.steps, warmup, args.seed)
    clock_info = clocks.stop()
    value = args.batch * 1000.0 / ms
    spread = decode_device_time.spread

    e2e, h2d, d2h = decode_e2e(eng, args.batch, args.prompt_len, args.steps, args.seed + 1)

    weight_bytes = cfg.weight_bytes_per_decode_step(2)
    kv_bytes = args.batch * mean_ctx * cfg.kv_bytes_per_token(2)
    achieved = (weight_bytes + kv_bytes) / (ms * 1e-3) / 1e9

    attn_flops = cfg.num_hidden_layers * 4 * cfg.q_dim * (T * (T + 1) // 2)
    pf_flops = cfg.matmul_flops_per_token() * T + attn_flops + 2 * cfg.vocab_size * cfg.hidden_size
    prefill = {"value": T / (pf_ms * 1e-3), "tokens": T, "ms": pf_ms, "frac": pf_flops / (pf_ms * 1e-3) / (bf16_tflops * 1e12)}

    points = {}
    if not args.no_points:
        for b in (1, 64):
            pms, _, _ = decode_device_time(eng, b, args.prompt_len, min(args.steps, 128), warmup, args.seed + 3 + b)
            points[f"decode_b{b}"] = b * 1000.0 / pms

    line = {
        "metric": "decode tok/s @ batch 8; Qwen3-4B shape BF16 (points: batch 1/64; prefill tok/s @ 2048 tok)",
        "value": value, "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded uniform token ids, random normal(0,0.02) weights", "impl": "ours",
        "config": {
            "model": args.preset, "layers": cfg.num_hidden_layers, "layers_of_shape": full_layers,
            "hidden": cfg.hidden_size, "q_heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
            "tied_head": cfg.tie_word_embeddings, "global_batch": args.batch, "seq_len": args.prompt_len,
            "mean_context": mean_ctx, "max_context": raw["max_position_embeddings"], "page_size": 64,
            "parallelism": "single-gpu", "cuda_graphs": True, "l2": "inputs>L2 (8 GB of weights per step)",
            "peaks": peak_src, **({"engine_opts": ",".join(args.engine_opt)} if args.engine_opt else {}),
        },
        "e2e": {"value": e2e, "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        # as hari495/dryft's harness reports them (agent/bench.py:58-59,86-87): (slowest - fastest) / median over the
        # eighths of the timed region, and the allocator's peaks over the whole run (weights, cache for batch 64, prompts)
        "spread": spread,
        "peak_mem_gib": {"allocated": torch.cuda.max_memory_allocated() / 2**30, "reserved": torch.cuda.max_memory_reserved() / 2**30},
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_gbs, "unit": "GB/s", "frac": achieved / hbm_gbs},
        "points": points,
        "clocks": clock_info,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
