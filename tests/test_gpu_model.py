"""The engine against the plain implementation, in 32-bit and in bfloat16: each request alone and
whole; with the last 32 tokens one by one; in batches of unequal lengths whose shorter requests end
earlier, batch after batch so that slots are used again; long decoding; the first tokens of a
sequence; generation through the entry point; parts alone; and a toy mixer with state of its own that
is registered, built and stepped without touching the library's files."""

import math

import pytest
import torch

import helpers as H
import plain_qwen3 as P

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
NAMES = ["a", "b", "c", "d"]

_engines = {}
_plains = {}


def engine_for(model_dirs, name, dtype, **kw):
    from dryft_b200.engine.api import Engine

    key = (name, dtype, tuple(sorted(kw.items())))
    if key not in _engines:
        opts = dict(dtype=dtype, max_batch=4, max_seq_len=512, max_tokens=4 * 512)
        opts.update(kw)
        _engines[key] = Engine(model_dirs[name], **opts)
    return _engines[key]


def plain_for(model_dirs, name, dtype):
    key = (name, dtype)
    if key not in _plains:
        _plains[key] = P.load_plain(model_dirs[name], dtype)
    return _plains[key]


def check(got: torch.Tensor, name, tokens, rows, model_dirs, dtype, what=""):
    """got [len(rows), V] vs the plain logits of the whole sequence at ``rows``."""
    p32 = plain_for(model_dirs, name, torch.float32).logits(tokens)[rows]
    got = got.float().cpu()
    assert torch.isfinite(got).all(), what
    if dtype == torch.float32:
        e = H.rel_err(got, p32)
        assert e <= H.FP32_TOL, f"{what}: 32-bit logits off by {e:.3g}"
    else:
        pb = plain_for(model_dirs, name, torch.bfloat16).logits(tokens)[rows]
        tol = H.bf16_tol(pb, p32)
        e = H.rel_err(got, pb)
        assert e <= tol, f"{what}: bfloat16 logits off by {e:.3g} (allowed {tol:.3g})"


def step(eng, slots, tokens, want):
    with torch.inference_mode():
        return eng.stepper.step(slots, tokens, want)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_requests_alone(model_dirs, name, dtype):
    eng = engine_for(model_dirs, name, dtype)
    for i, n in enumerate([1, 2, 7, 31, 64, 65, 150]):
        toks = H.prompts_for(name, [n], seed=i)[0]
        (slot,) = eng.cache.open_sequences(1)
        got = step(eng, [slot], [toks], [list(range(n))])
        eng.cache.close_sequences([slot])
        check(got, name, toks, list(range(n)), model_dirs, dtype, f"{name} whole len {n}")
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_last_32_tokens_one_by_one(model_dirs, name, dtype):
    eng = engine_for(model_dirs, name, dtype)
    for i, n in enumerate([33, 40, 100, 160]):
        toks = H.prompts_for(name, [n], seed=10 + i)[0]
        head = n - 32
        (slot,) = eng.cache.open_sequences(1)
        rows = [step(eng, [slot], [toks[:head]], [[head - 1]])]
        for t in range(head, n):
            rows.append(step(eng, [slot], [[toks[t]]], [[0]]))
        eng.cache.close_sequences([slot])
        got = torch.cat(rows)
        check(got, name, toks, list(range(head - 1, n)), model_dirs, dtype, f"{name} len {n} last 32 one by one")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_one_after_another(model_dirs, name, dtype):
    """Requests of unequal total lengths start together with unequal prompts, go on one token each,
    the shorter ones end earlier; three batches in a row on 4 slots so every slot is used again (the
    second batch's sequences are longer than the first's, so stale keys would be seen if lengths
    leaked)."""
    eng = engine_for(model_dirs, name, dtype)
    batches = [
        [(5, 9), (13, 13), (1, 4)],             # (prompt length, total length)
        [(31, 70), (7, 75), (16, 20), (64, 66)],
        [(3, 40), (65, 67)],
    ]
    seed = 100
    for bi, batch in enumerate(batches):
        seqs = []
        for (pl, tl) in batch:
            seed += 1
            seqs.append(H.prompts_for(name, [tl], seed=seed)[0])
        slots = eng.cache.open_sequences(len(batch))
        got = {i: [] for i in range(len(batch))}
        rows_of = {i: [] for i in range(len(batch))}
        out = step(eng, slots, [s[:pl] for s, (pl, _) in zip(seqs, batch)], [[pl - 1] for (pl, _) in batch])
        for i, (pl, _) in enumerate(batch):
            got[i].append(out[i:i + 1])
            rows_of[i].append(pl - 1)
        fed = [pl for (pl, _) in batch]
        alive = [i for i, (pl, tl) in enumerate(batch) if pl < tl]
        ended = [i for i in range(len(batch)) if i not in alive]
        eng.cache.close_sequences([slots[i] for i in ended])  # ends right after its prompt
        while alive:
            out = step(eng, [slots[i] for i in alive], [[seqs[i][fed[i]]] for i in alive], [[0] for _ in alive])
            for j, i in enumerate(alive):
                got[i].append(out[j:j + 1])
                rows_of[i].append(fed[i])
                fed[i] += 1
            done = [i for i in alive if fed[i] >= batch[i][1]]
            eng.cache.close_sequences([slots[i] for i in done])
            alive = [i for i in alive if i not in done]
        for i in range(len(batch)):
            check(torch.cat(got[i]), name, seqs[i], rows_of[i], model_dirs, dtype, f"{name} batch {bi} request {i}")
        eng.cache.check()
    assert eng.cache.slots.n_held == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["a", "c"])
def test_long_decoding(model_dirs, name, dtype):
    """A short prompt and 300 decoded tokens: crosses several pages and, for the windowed
    configuration, leaves the window far behind."""
    eng = engine_for(model_dirs, name, dtype)
    n = 305
    toks = H.prompts_for(name, [n], seed=77)[0]
    (slot,) = eng.cache.open_sequences(1)
    rows = [step(eng, [slot], [toks[:5]], [[4]])]
    for t in range(5, n):
        rows.append(step(eng, [slot], [[toks[t]]], [[0]]))
    eng.cache.close_sequences([slot])
    check(torch.cat(rows), name, toks, list(range(4, n)), model_dirs, dtype, f"{name} long decoding")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_first_tokens_of_a_sequence(model_dirs, name, dtype):
    """A one-token prompt, then tokens one by one: positions 0, 1, 2, ... with nothing before them."""
    eng = engine_for(model_dirs, name, dtype)
    toks = H.prompts_for(name, [6], seed=5)[0]
    (slot,) = eng.cache.open_sequences(1)
    rows = [step(eng, [slot], [[t]], [[0]]) for t in toks]
    eng.cache.close_sequences([slot])
    check(torch.cat(rows), name, toks, list(range(6)), model_dirs, dtype, f"{name} first tokens")


@pytest.mark.parametrize("name", NAMES)
def test_cutting_invariance_32bit(model_dirs, name):
    """In 32-bit the same request gives the same logits (to rounding) whole, in two chunks, and
    inside a batch with other requests."""
    eng = engine_for(model_dirs, name, torch.float32)
    toks = H.prompts_for(name, [90], seed=31)[0]
    other = H.prompts_for(name, [17, 130], seed=32)
    s = eng.cache.open_sequences(1)
    whole = step(eng, s, [toks], [list(range(90))]).cpu()
    eng.cache.close_sequences(s)
    s = eng.cache.open_sequences(1)
    a = step(eng, s, [toks[:37]], [list(range(37))]).cpu()
    b = step(eng, s, [toks[37:]], [list(range(53))]).cpu()
    eng.cache.close_sequences(s)
    assert H.rel_err(torch.cat([a, b]), whole) <= H.FP32_TOL
    s = eng.cache.open_sequences(3)
    out = step(eng, s, [other[0], toks, other[1]], [[], list(range(90)), [0]]).cpu()
    eng.cache.close_sequences(s)
    assert H.rel_err(out[:90], whole) <= H.FP32_TOL


# ----------------------------------------------------------------------------- the entry point
def _margins(plain, prompt, ours):
    """Teacher-forced margin of each of our tokens under the plain model: max logit - logit[ours]
    (the reference's replay margin, agent/verify.py:100-109)."""
    lg = plain.logits(list(prompt) + list(ours[:-1]))[len(prompt) - 1:]
    best = lg.max(dim=-1).values
    mine = lg.gather(1, torch.tensor(ours)[:, None])[:, 0]
    return (best - mine), lg


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,lengths,steps", [("a", [5, 9, 13], 8), ("b", [1, 7, 16, 31], 12), ("c", [30, 3], 50)])
def test_greedy_generation_through_entry_point(model_dirs, name, lengths, steps, dtype):
    eng = engine_for(model_dirs, name, dtype)
    prompts = H.prompts_for(name, lengths, seed=3)
    out = [s for s in eng.generate(prompts, steps)]
    assert len(out) == steps and all(len(s) == len(prompts) for s in out)
    again = [s for s in eng.generate(prompts, steps)]
    assert again == out, "second run differs from the first (stale state)"
    plain = plain_for(model_dirs, name, torch.float32)
    for b, p in enumerate(prompts):
        ours = [s[b] for s in out]
        if dtype == torch.float32:
            want = P.plain_generate(plain, [p], steps)[0]
            assert ours == want, f"{name} sequence {b}"
        else:
            m, lg = _margins(plain, p, ours)
            assert float(m.max()) <= 0.05 * float(lg.abs().max()), f"{name} sequence {b}: margin {float(m.max()):.3g}"
    eng.cache.check()
    assert eng.cache.slots.n_held == 0


def test_sampled_generation_matches_plain(model_dirs):
    """Config B's workload: 4 prompts of 1/7/16/31 tokens, 12 steps at temperature 0.7, top-k 20."""
    eng = engine_for(model_dirs, "b", torch.float32)
    prompts = H.prompts_for("b", [1, 7, 16, 31], seed=9)
    out = [s for s in eng.generate(prompts, 12, temperature=0.7, top_k=20, seed=42)]
    plain = plain_for(model_dirs, "b", torch.float32)
    want = P.plain_generate(plain, prompts, 12, temperature=0.7, top_k=20, seed=42)
    for b in range(4):
        assert [s[b] for s in out] == want[b]
    # the draws of a sequence do not depend on the batch it is in
    alone = [s[0] for s in eng.generate([prompts[2]], 12, temperature=0.7, top_k=20, seed=42)]
    assert alone == P.plain_generate(plain, [prompts[2]], 12, temperature=0.7, top_k=20, seed=42)[0]


def test_stop_tokens_and_batches_in_a_row(model_dirs):
    """More requests than slots, stop tokens that end some sequences early: -1 afterwards, slots
    reused by the next batch, results equal to the plain model's."""
    eng = engine_for(model_dirs, "a", torch.float32)
    plain = plain_for(model_dirs, "a", torch.float32)
    prompts = H.prompts_for("a", [4, 11, 2, 19, 6, 33, 9, 5, 12, 3], seed=21)
    free_run = P.plain_generate(plain, prompts, 10)
    stops = sorted({free_run[1][3], free_run[4][0], free_run[7][6]})
    want = P.plain_generate(plain, prompts, 10, stop_token_ids=stops)
    got = eng.generate_many(prompts, 10, stop_token_ids=stops)
    assert got == want
    steps = [s for s in eng.generate(prompts[:4], 10, stop_token_ids=stops)]
    for b in range(4):
        col = [s[b] for s in steps]
        n = len(want[b])
        assert col[:n] == want[b] and all(t == -1 for t in col[n:])
    eng.cache.check()
    assert eng.cache.slots.n_held == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_cuda_graph_decode_equals_eager(model_dirs, dtype):
    g = engine_for(model_dirs, "b", dtype)
    e = engine_for(model_dirs, "b", dtype, cuda_graphs=False)
    prompts = H.prompts_for("b", [9, 2, 40], seed=8)
    a = [s for s in g.generate(prompts, 20)]
    b = [s for s in e.generate(prompts, 20)]
    assert a == b
    # sequences leaving mid-way change the padded batch: still equal
    stop = [a[5][1]]
    assert [s for s in g.generate(prompts, 20, stop_token_ids=stop)] == [s for s in e.generate(prompts, 20, stop_token_ids=stop)]


def test_fused_decode_products_equal_the_separate_kernels(model_dirs):
    """With few rows the norms, residual adds and SiLU*mul are folded into the matrix products and
    launched as programmatic dependents; the logits must stay those of the separate kernels (same
    rounding points, sums in another order), and switching the launch overlap off changes no bit."""
    fused = engine_for(model_dirs, "b", torch.bfloat16)
    plain_launch = engine_for(model_dirs, "b", torch.bfloat16, pdl=False)
    separate = engine_for(model_dirs, "b", torch.bfloat16, fuse_decode=False)
    toks = H.prompts_for("b", [40], seed=12)[0]
    outs = []
    for eng in (fused, plain_launch, separate):
        s = eng.cache.open_sequences(1)
        rows = [step(eng, s, [toks[:30]], [[29]])]
        for t in toks[30:]:
            rows.append(step(eng, s, [[t]], [[0]]))
        eng.cache.close_sequences(s)
        outs.append(torch.cat(rows).float().cpu())
    assert torch.equal(outs[0], outs[1])
    p32 = plain_for(model_dirs, "b", torch.float32).logits(toks)[29:]
    pb = plain_for(model_dirs, "b", torch.bfloat16).logits(toks)[29:]
    assert H.rel_err(outs[0], outs[2]) <= H.bf16_tol(pb, p32)
    from dryft_b200.ops import kernels as K
    K.check_error_flags()


def test_norm_split_over_two_launches(model_dirs):
    """An option (``norm_ahead=True``; off by default): at widths that are multiples of 256 a fused decode product
    leaves the stream weighted for the next norm and the product behind that norm scales its sums instead of
    normalising its input -- the activations are then rounded once where the reference rounds twice
    (``engine/dryft_qwen3/model.py:28-32``).  Measured on this configuration and at the Qwen3-4B widths (2 and 8
    layers): the option's logits are as close to the plain 32-bit ones as the default's (0.98 to 1.09 times its
    error) and up to 1.36 times as far from the plain bfloat16 ones.  Asserted here: the option runs (other bits),
    stays within those factors, and the default stays within bfloat16 rounding of the plain implementation;
    CUDA-graph decoding gives the same tokens as eager decoding with the option on."""
    on = engine_for(model_dirs, "d", torch.bfloat16, norm_ahead=True)
    off = engine_for(model_dirs, "d", torch.bfloat16)
    assert off.rt.norm_ahead is False, "the default path keeps the reference's rounding points"
    errs = {"on": [], "off": []}
    differs = False
    p32m, pbm = plain_for(model_dirs, "d", torch.float32), plain_for(model_dirs, "d", torch.bfloat16)
    for seed in (21, 22, 23):
        toks = H.prompts_for("d", [60], seed=seed)[0]
        p32, pb = p32m.logits(toks)[27:], pbm.logits(toks)[27:]
        tol = H.bf16_tol(pb, p32)
        outs = {}
        for name, eng in (("on", on), ("off", off)):
            s = eng.cache.open_sequences(1)
            rows = [step(eng, s, [toks[:28]], [[27]])]
            for t in toks[28:]:
                rows.append(step(eng, s, [[t]], [[0]]))
            eng.cache.close_sequences(s)
            outs[name] = torch.cat(rows).float().cpu()
            errs[name].append((H.rel_err(outs[name], pb), H.rel_err(outs[name], p32)))
            assert H.rel_err(outs[name], pb) <= tol
        differs = differs or not torch.equal(outs["on"], outs["off"])
    assert differs, "the split path did not run"
    on_b, off_b = max(e[0] for e in errs["on"]), max(e[0] for e in errs["off"])
    on_32, off_32 = max(e[1] for e in errs["on"]), max(e[1] for e in errs["off"])
    assert on_32 <= 1.25 * off_32, f"the option is further from 32-bit than measured: {on_32:.4f} vs {off_32:.4f}"
    assert on_b <= 1.6 * off_b, f"the option is further from plain bfloat16 than measured: {on_b:.4f} vs {off_b:.4f}"
    prompts = H.prompts_for("d", [9, 2, 40], seed=8)
    eager = engine_for(model_dirs, "d", torch.bfloat16, cuda_graphs=False, norm_ahead=True)
    assert [s for s in on.generate(prompts, 16)] == [s for s in eager.generate(prompts, 16)]
    from dryft_b200.ops import kernels as K
    K.check_error_flags()


def test_requests_beyond_capacity_are_refused(model_dirs):
    eng = engine_for(model_dirs, "a", torch.float32)
    with pytest.raises(ValueError):
        list(eng.generate(H.prompts_for("a", [3] * 5), 4))           # more sequences than max_batch
    with pytest.raises(ValueError):
        list(eng.generate(H.prompts_for("a", [500]), 100))           # longer than max_seq_len
    with pytest.raises(ValueError):
        list(eng.generate([[1, 2], []], 4))                          # empty prompt
    with pytest.raises(ValueError):
        list(eng.generate([[1, 999999]], 4))                         # token outside the vocabulary
    assert list(eng.generate([], 4)) == [] and list(eng.generate([[1]], 0)) == []
    eng.cache.check()
    assert eng.cache.slots.n_held == 0


# ----------------------------------------------------------------------------- parts alone
@pytest.mark.parametrize("dtype", DTYPES)
def test_parts_alone(dtype):
    """Norm, feed-forward and attention mixer built from specs at sizes of their own (not a model's),
    against the plain functions."""
    from dryft_b200.cache.store import SequenceCache
    from dryft_b200.config.spec import PartSpec
    from dryft_b200.ops import kernels as K
    from dryft_b200.parts import FFNS, MIXERS, NORMS, Runtime, StepContext
    from dryft_b200.parts.base import TensorInfo
    from dryft_b200.weights import RandomSource

    dev = torch.device("cuda:0")
    rt = Runtime(dtype=dtype, device=dev, sm_count=torch.cuda.get_device_properties(dev).multi_processor_count)
    hidden, inter, nh, nkv, d = 72, 200, 6, 3, 32
    attn_params = {"hidden_size": hidden, "num_heads": nh, "num_kv_heads": nkv, "head_dim": d, "scale": 0.2,
                   "window": None, "qk_norm": PartSpec("rmsnorm", {"size": d, "eps": 1e-5}),
                   "position": PartSpec("rope", {"rotary_dim": d, "theta": 12345.0})}
    ffn_params = {"hidden_size": hidden, "intermediate_size": inter}
    norm_params = {"size": hidden, "eps": 2e-6}
    exp = {}
    exp.update(NORMS.get("rmsnorm").tensors(norm_params, "n."))
    exp.update(FFNS.get("swiglu").tensors(ffn_params, "f."))
    exp.update(MIXERS.get("attention").tensors(attn_params, "m."))
    src = RandomSource(exp, 5, dtype, dev, std=0.1)
    cpu = {n: src._read(n).cpu() for n in exp}
    cpu = {n: (t.float() if dtype == torch.float32 else t) for n, t in cpu.items()}
    tol = 3e-2 if dtype == torch.bfloat16 else 1e-4
    with torch.inference_mode():
        norm = NORMS.get("rmsnorm")(norm_params, "n.", src, rt)
        ffn = FFNS.get("swiglu")(ffn_params, "f.", src, rt)
        mixer = MIXERS.get("attention")(attn_params, "m.", src, rt)
        x = torch.randn(21, hidden, device=dev).to(dtype)
        torch.testing.assert_close(norm.forward(x).cpu().float(), P.rmsnorm(x.cpu(), cpu["n.weight"], 2e-6).float(), rtol=tol, atol=tol)
        got = ffn.forward(x, None).cpu().float()
        ref = P.swiglu(x.cpu(), cpu["f.gate_proj.weight"], cpu["f.up_proj.weight"], cpu["f.down_proj.weight"], dtype).float()
        torch.testing.assert_close(got, ref, rtol=tol, atol=tol)
        # the mixer over two sequences (13 and 8 tokens) in one step, through a cache of its own
        cache = SequenceCache([(mixer.kv_need(), None)], [None], max_tokens=256, max_slots=2, max_seq_len=128,
                              page_size=64, dtype=dtype, device=dev)
        slots = cache.open_sequences(2)
        lens = [13, 8]
        for s, n in zip(slots, lens):
            cache.reserve(s, n)
        cache.flush()
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        cu, tok_slot, tok_pos = i32([0, 13, 21]), torch.empty(21, dtype=torch.int32, device=dev), torch.empty(21, dtype=torch.int32, device=dev)
        K.step_meta(cu, i32(slots), cache.seq_len, tok_slot, tok_pos, 21, 2)
        ctx = StepContext(n_tokens=21, n_seqs=2, tokens=i32([0] * 21), cu_q=cu, seq_slot=i32(slots), tok_slot=tok_slot,
                          tok_pos=tok_pos, decode=False, max_kv=13, tile_tok0=i32([0, 13]), tile_rows=i32([13, 8]), n_tiles=2, tile_size=64)
        got = mixer.forward(x, ctx, cache.entry(0), None, True).cpu().float()
        refs = []
        for lo, n in ((0, 13), (13, 8)):
            h = x[lo:lo + n].cpu()
            q = P.matmul_nt(h, cpu["m.q_proj.weight"], dtype).view(n, nh, d)
            k = P.matmul_nt(h, cpu["m.k_proj.weight"], dtype).view(n, nkv, d)
            v = P.matmul_nt(h, cpu["m.v_proj.weight"], dtype).view(n, nkv, d)
            q = P.rmsnorm(q, cpu["m.q_norm.weight"], 1e-5)
            k = P.rmsnorm(k, cpu["m.k_norm.weight"], 1e-5)
            cos, sin = P.rope_cos_sin(torch.arange(n), d, 12345.0, dtype)
            o = P.causal_attention(P.apply_rope(q, cos, sin), P.apply_rope(k, cos, sin), v, 0.2, None, dtype)
            refs.append(P.matmul_nt(o, cpu["m.o_proj.weight"], dtype).float())
        torch.testing.assert_close(got, torch.cat(refs), rtol=tol, atol=tol)


# ----------------------------------------------------------------------------- a toy mixer with state
def test_toy_mixer_with_state_registers_builds_and_steps():
    """A mixer that keeps a running sum of its inputs per sequence (fixed-size state, no keys or
    values), defined here, registered under a new kind, put into a new architecture whose layers
    alternate it with attention, built with random weights and stepped — whole prompts, token by
    token, and on a reused slot — without a change to any file of the library."""
    from dryft_b200.cache.store import StateNeed
    from dryft_b200.config import register_architecture, unregister_architecture
    from dryft_b200.config.spec import LayerSpec, ModelSpec, PartSpec, RunStep
    from dryft_b200.engine.api import Engine
    from dryft_b200.parts import MIXERS, TensorInfo, register_mixer
    from dryft_b200.parts.linear import linear

    class RunningMean:
        @staticmethod
        def tensors(params, prefix):
            return {prefix + "mix.weight": TensorInfo((params["hidden_size"], params["hidden_size"]), "matrix")}

        def __init__(self, params, prefix, weights, rt):
            self.rt = rt
            self.hidden = params["hidden_size"]
            self.w = weights.load(prefix + "mix.weight", "matrix")

        def kv_need(self):
            return None

        def state_need(self):
            return StateNeed((self.hidden,), torch.float32)

        def forward(self, h, ctx, cache, state, owns_cache=True):
            # mean of the sequence's inputs up to and including each token; the running sum is the state
            out = torch.zeros_like(h, dtype=torch.float32)
            cu = ctx.cu_q.tolist()
            slots = ctx.seq_slot.tolist()
            for b, slot in enumerate(slots):
                if slot < 0:
                    continue
                rows = h[cu[b]:cu[b + 1]].float()
                sums = state[slot][None, :] + torch.cumsum(rows, dim=0)
                pos = ctx.tok_pos[cu[b]:cu[b + 1]].float()[:, None]
                out[cu[b]:cu[b + 1]] = sums / (pos + 1.0)
                state[slot] = sums[-1]
            return linear(out.to(h.dtype), self.w, self.rt)

    class ToyConfig:
        def __init__(self, raw):
            self.raw = dict(raw)

        def to_dict(self):
            return dict(self.raw)

        def model_spec(self):
            r = self.raw
            H_, V = r["hidden_size"], r["vocab_size"]
            norm = PartSpec("rmsnorm", {"size": H_, "eps": 1e-6})
            attn = PartSpec("attention", {"hidden_size": H_, "num_heads": 2, "num_kv_heads": 1, "head_dim": 16,
                                          "scale": 0.25, "window": None, "qk_norm": None,
                                          "position": PartSpec("rope", {"rotary_dim": 8, "theta": 100.0})})
            toy = PartSpec("toy_running_mean", {"hidden_size": H_})
            ffn = PartSpec("swiglu", {"hidden_size": H_, "intermediate_size": 48})
            layers = tuple(LayerSpec("prenorm", m, ffn, norm, norm, f"l{i}.mixer.", f"l{i}.ffn.", f"l{i}.n1.", f"l{i}.n2.")
                           for i, m in enumerate([toy, attn, toy]))
            # run order names layer 0 twice (shared weights, separate state)
            sched = (RunStep(0), RunStep(1), RunStep(2), RunStep(0))
            return ModelSpec("ToyForCausalLM", V, H_, 256, PartSpec("embedding", {"vocab_size": V, "hidden_size": H_}),
                             layers, sched, norm, PartSpec("lm_head", {"vocab_size": V, "hidden_size": H_, "tied": True}),
                             embedding_prefix="emb.", final_norm_prefix="fn.", head_prefix="head.")

    register_mixer("toy_running_mean", RunningMean)
    register_architecture("ToyForCausalLM", ToyConfig)
    try:
        raw = {"architectures": ["ToyForCausalLM"], "hidden_size": 32, "vocab_size": 97}
        eng = Engine.from_config(raw, seed=3, std=0.2, dtype="float32", max_batch=2, max_seq_len=128, max_tokens=256)
        toks = torch.randint(0, 97, (20,), generator=torch.Generator().manual_seed(0)).tolist()
        with torch.inference_mode():
            s = eng.cache.open_sequences(1)
            whole = eng.stepper.step(s, [toks], [list(range(20))]).cpu()
            eng.cache.close_sequences(s)
            # same slot again (reuse): the state must start from zero; feed in pieces
            s2 = eng.cache.open_sequences(1)
            assert s2 == s
            parts = [eng.stepper.step(s2, [toks[:7]], [list(range(7))]).cpu()]
            for t in toks[7:]:
                parts.append(eng.stepper.step(s2, [[t]], [[0]]).cpu())
            eng.cache.close_sequences(s2)
            # and as one of two sequences in a batch
            s3 = eng.cache.open_sequences(2)
            both = eng.stepper.step(s3, [toks[:5], toks], [[], list(range(20))]).cpu()
            eng.cache.close_sequences(s3)
        assert torch.isfinite(whole).all() and float(whole.abs().max()) > 0
        assert H.rel_err(torch.cat(parts), whole) <= H.FP32_TOL
        assert H.rel_err(both, whole) <= H.FP32_TOL
        # the state matters: the logits at the last place depend on the first token
        with torch.inference_mode():
            s = eng.cache.open_sequences(1)
            other = eng.stepper.step(s, [[(toks[0] + 1) % 97] + toks[1:]], [[19]]).cpu()
            eng.cache.close_sequences(s)
        assert H.rel_err(other, whole[19:20]) > 1e-3
    finally:
        MIXERS.unregister("toy_running_mean")
        unregister_architecture("ToyForCausalLM")


@pytest.mark.gpu
def test_layer_reading_another_layers_cache():
    """A run order in which one attention layer keeps no keys of its own and reads the cache that an
    earlier layer wrote in the same step (queries only are projected there).  Whole prompts, the last
    tokens one by one (the one-launch decode attention without a cache write, which must see the other
    layer's write of this very step), a batch of two, and graph-captured decoding must agree."""
    from dryft_b200.config import register_architecture, unregister_architecture
    from dryft_b200.config.spec import LayerSpec, ModelSpec, PartSpec, RunStep
    from dryft_b200.engine.api import Engine

    class SharedKVConfig:
        def __init__(self, raw):
            self.raw = dict(raw)

        def to_dict(self):
            return dict(self.raw)

        def model_spec(self):
            r = self.raw
            H_, V = r["hidden_size"], r["vocab_size"]
            norm = PartSpec("rmsnorm", {"size": H_, "eps": 1e-6})
            attn = PartSpec("attention", {"hidden_size": H_, "num_heads": 4, "num_kv_heads": 2, "head_dim": 32,
                                          "scale": 32 ** -0.5, "window": None,
                                          "qk_norm": PartSpec("rmsnorm", {"size": 32, "eps": 1e-6}),
                                          "position": PartSpec("rope", {"rotary_dim": 32, "theta": 1e4})})
            ffn = PartSpec("swiglu", {"hidden_size": H_, "intermediate_size": 96})
            layers = tuple(LayerSpec("prenorm", attn, ffn, norm, norm, f"l{i}.attn.", f"l{i}.ffn.", f"l{i}.n1.", f"l{i}.n2.")
                           for i in range(3))
            sched = (RunStep(0), RunStep(1, cache_from=0), RunStep(2))
            return ModelSpec("SharedKVForCausalLM", V, H_, 512, PartSpec("embedding", {"vocab_size": V, "hidden_size": H_}),
                             layers, sched, norm, PartSpec("lm_head", {"vocab_size": V, "hidden_size": H_, "tied": True}),
                             embedding_prefix="emb.", final_norm_prefix="fn.", head_prefix="head.")

    register_architecture("SharedKVForCausalLM", SharedKVConfig)
    try:
        raw = {"architectures": ["SharedKVForCausalLM"], "hidden_size": 64, "vocab_size": 211}
        n = 150
        toks = torch.randint(0, 211, (n,), generator=torch.Generator().manual_seed(1)).tolist()
        whole32 = None
        for dtype in ("float32", "bfloat16"):
            eng = Engine.from_config(raw, seed=5, std=0.15, dtype=dtype, max_batch=2, max_seq_len=512, max_tokens=1024)
            with torch.inference_mode():
                s = eng.cache.open_sequences(1)
                whole = eng.stepper.step(s, [toks], [list(range(n))]).cpu()
                eng.cache.close_sequences(s)
                s = eng.cache.open_sequences(1)
                parts = [eng.stepper.step(s, [toks[:n - 32]], [list(range(n - 32))]).cpu()]
                for t in toks[n - 32:]:
                    parts.append(eng.stepper.step(s, [[t]], [[0]]).cpu())
                eng.cache.close_sequences(s)
                s = eng.cache.open_sequences(2)
                both = eng.stepper.step(s, [toks[:40], toks], [[39], list(range(n))]).cpu()
                eng.cache.close_sequences(s)
            if dtype == "float32":
                whole32, tol = whole, H.FP32_TOL
            else:
                tol = H.bf16_tol(whole, whole32)   # what bfloat16 rounding alone does to these logits, doubled
            assert torch.isfinite(whole).all()
            assert H.rel_err(torch.cat(parts), whole) <= tol
            assert H.rel_err(both[1:], whole) <= tol and H.rel_err(both[:1], whole[39:40]) <= tol
            # greedy generation (graph-captured decode from the device state) equals stepping by hand
            out = eng.generate_many([toks[:50], toks[:9]], max_new_tokens=12)
            with torch.inference_mode():
                for prompt, got in zip((toks[:50], toks[:9]), out):
                    # our tokens fed back by hand, one sequence alone: each must be the best choice of that step's
                    # logits -- exactly in 32-bit, up to the measured bfloat16 noise of these logits otherwise
                    s = eng.cache.open_sequences(1)
                    lg = eng.stepper.step(s, [prompt], [[len(prompt) - 1]])
                    for t in got:
                        margin = float(lg[0].max() - lg[0][t])
                        if dtype == "float32":
                            assert margin <= 2 * H.FP32_TOL * float(lg.abs().max()), f"token {t} is not the 32-bit choice"
                        else:
                            assert margin <= tol * float(lg.abs().max()), f"token {t} loses {margin:.3g} to the best"
                        lg = eng.stepper.step(s, [[t]], [[0]])
                    eng.cache.close_sequences(s)
            del eng
    finally:
        unregister_architecture("SharedKVForCausalLM")


@pytest.mark.gpu
def test_toy_routed_ffn_and_toy_position_encoding_register_build_and_step():
    """Two more parts defined here and registered without a change to the library: a feed-forward that
    routes every token to one of three small experts (router logits in 32-bit, first index on ties) and a
    rotary position encoding with interpolated positions (angles = pos / factor * inv_freq).  A new
    architecture uses them in different layers (the first layer keeps the stock parts); whole prompts,
    token by token, two sequences in a batch, and a plain evaluation written out here must agree."""
    from dryft_b200.config import register_architecture, unregister_architecture
    from dryft_b200.config.spec import LayerSpec, ModelSpec, PartSpec, RunStep
    from dryft_b200.engine.api import Engine
    from dryft_b200.parts import FFNS, POSITIONS, TensorInfo, register_ffn, register_position
    from dryft_b200.parts.linear import linear

    n_exp, inter = 3, 40

    class RoutedFFN:
        @staticmethod
        def tensors(params, prefix):
            h = params["hidden_size"]
            t = {prefix + "router.weight": TensorInfo((n_exp, h), "matrix")}
            for e in range(n_exp):
                t[prefix + f"experts.{e}.up.weight"] = TensorInfo((inter, h), "matrix")
                t[prefix + f"experts.{e}.down.weight"] = TensorInfo((h, inter), "matrix")
            return t

        def __init__(self, params, prefix, weights, rt):
            self.rt = rt
            self.router = weights.load(prefix + "router.weight", "matrix")
            self.up = [weights.load(prefix + f"experts.{e}.up.weight", "matrix") for e in range(n_exp)]
            self.down = [weights.load(prefix + f"experts.{e}.down.weight", "matrix") for e in range(n_exp)]

        def forward(self, h, ctx):
            logits = h.float() @ self.router.float().T          # router logits in 32-bit
            choice = logits.argmax(dim=-1)                       # first index on ties
            out = torch.zeros_like(h)
            for e in range(n_exp):
                rows = (choice == e).nonzero(as_tuple=True)[0]
                if rows.numel():
                    a = torch.relu(linear(h[rows].contiguous(), self.up[e], self.rt))
                    out[rows] = linear(a, self.down[e], self.rt)
            return out

    class InterpolatedRope:
        def __init__(self, params, head_dim, rt):
            self.rotary_dim = int(params["rotary_dim"])
            r = self.rotary_dim
            inv = 1.0 / (float(params["theta"]) ** (torch.arange(0, r, 2, dtype=torch.int64).to(torch.float32) / r))
            self.inv_freq = (inv / float(params["factor"])).to(rt.device)

    class ToyConfig:
        def __init__(self, raw):
            self.raw = dict(raw)

        def to_dict(self):
            return dict(self.raw)

        def model_spec(self):
            r = self.raw
            H_, V = r["hidden_size"], r["vocab_size"]
            norm = PartSpec("rmsnorm", {"size": H_, "eps": 1e-5})

            def attn(pos):
                return PartSpec("attention", {"hidden_size": H_, "num_heads": 3, "num_kv_heads": 3, "head_dim": 16,
                                              "scale": 0.25, "window": None, "qk_norm": None, "position": pos})
            stock_pos = PartSpec("rope", {"rotary_dim": 16, "theta": 1e4})
            toy_pos = PartSpec("toy_interpolated_rope", {"rotary_dim": 16, "theta": 1e4, "factor": 4.0})
            dense = PartSpec("swiglu", {"hidden_size": H_, "intermediate_size": 64})
            routed = PartSpec("toy_routed", {"hidden_size": H_})
            parts = [(attn(stock_pos), dense), (attn(toy_pos), routed), (attn(toy_pos), dense)]
            layers = tuple(LayerSpec("prenorm", m, f, norm, norm, f"l{i}.attn.", f"l{i}.ffn.", f"l{i}.n1.", f"l{i}.n2.")
                           for i, (m, f) in enumerate(parts))
            return ModelSpec("ToyRoutedForCausalLM", V, H_, 256, PartSpec("embedding", {"vocab_size": V, "hidden_size": H_}),
                             layers, tuple(RunStep(i) for i in range(3)), norm,
                             PartSpec("lm_head", {"vocab_size": V, "hidden_size": H_, "tied": False}),
                             embedding_prefix="emb.", final_norm_prefix="fn.", head_prefix="head.")

    register_ffn("toy_routed", RoutedFFN)
    register_position("toy_interpolated_rope", InterpolatedRope)
    register_architecture("ToyRoutedForCausalLM", ToyConfig)
    try:
        raw = {"architectures": ["ToyRoutedForCausalLM"], "hidden_size": 48, "vocab_size": 131}
        eng = Engine.from_config(raw, seed=9, std=0.2, dtype="float32", max_batch=2, max_seq_len=128, max_tokens=256)
        n = 30
        toks = torch.randint(0, 131, (n,), generator=torch.Generator().manual_seed(2)).tolist()
        with torch.inference_mode():
            s = eng.cache.open_sequences(1)
            whole = eng.stepper.step(s, [toks], [list(range(n))]).cpu()
            eng.cache.close_sequences(s)
            s = eng.cache.open_sequences(1)
            parts = [eng.stepper.step(s, [toks[:11]], [list(range(11))]).cpu()]
            for t in toks[11:]:
                parts.append(eng.stepper.step(s, [[t]], [[0]]).cpu())
            eng.cache.close_sequences(s)
            s = eng.cache.open_sequences(2)
            both = eng.stepper.step(s, [toks, toks[:7]], [list(range(n)), [6]]).cpu()
            eng.cache.close_sequences(s)
        assert torch.isfinite(whole).all()
        assert H.rel_err(torch.cat(parts), whole) <= H.FP32_TOL
        assert H.rel_err(both[:n], whole) <= H.FP32_TOL and H.rel_err(both[n:], whole[6:7]) <= H.FP32_TOL

        # plain evaluation of the same model from the engine's own tensors, whole sequence, no cache
        m = eng.model
        x = P.embed(torch.tensor(toks), m.embedding.table.float().cpu(), torch.float32)
        pos = torch.arange(n)
        used = set()
        for blk, factor in zip(m.blocks, (1.0, 4.0, 4.0)):
            at, ff = blk.mixer, blk.ffn
            h = P.rmsnorm(x, blk.norm_mixer.weight.cpu(), 1e-5)
            qkv = h @ at.w_qkv.float().cpu().T
            q, k, v = (t.view(n, 3, 16) for t in qkv.split([48, 48, 48], dim=-1))
            inv = 1.0 / (1e4 ** (torch.arange(0, 16, 2, dtype=torch.int64).float() / 16)) / factor
            ang = pos.float()[:, None] * inv[None, :]
            cos, sin = torch.cat((ang.cos(), ang.cos()), -1)[:, None, :], torch.cat((ang.sin(), ang.sin()), -1)[:, None, :]
            rot = lambda t: t * cos + torch.cat((-t[..., 8:], t[..., :8]), -1) * sin
            q, k = rot(q), rot(k)
            sc = torch.einsum("qhd,khd->hqk", q, k) * 0.25
            sc = sc.masked_fill(torch.ones(n, n, dtype=torch.bool).triu(1), float("-inf"))
            o = torch.einsum("hqk,khd->qhd", torch.softmax(sc, -1), v).reshape(n, 48)
            x = x + o @ at.w_o.float().cpu().T
            h = P.rmsnorm(x, blk.norm_ffn.weight.cpu(), 1e-5)
            if hasattr(ff, "router"):
                choice = (h @ ff.router.float().cpu().T).argmax(-1)
                used |= set(choice.tolist())
                y = torch.stack([torch.relu(h[i] @ ff.up[int(e)].float().cpu().T) @ ff.down[int(e)].float().cpu().T
                                 for i, e in enumerate(choice)])
            else:
                gu = h @ ff.w_gate_up.float().cpu().T
                y = P.silu_mul(gu[:, :64], gu[:, 64:]) @ ff.w_down.float().cpu().T
            x = x + y
        logits = P.rmsnorm(x, m.final_norm.weight.cpu(), 1e-5) @ m.head.weight.float().cpu().T
        assert len(used) >= 2, "the routing must send tokens to different experts for the test to mean anything"
        assert H.rel_err(whole, logits) <= 5 * H.FP32_TOL
    finally:
        FFNS.unregister("toy_routed")
        POSITIONS.unregister("toy_interpolated_rope")
        unregister_architecture("ToyRoutedForCausalLM")


@pytest.mark.gpu
@pytest.mark.parametrize("n_seqs", [8, 12])
def test_decode_at_production_widths_is_the_same_with_and_without_launch_overlap(n_seqs):
    """Two layers at the widths the benchmark runs (hidden 2560, q width 4096, intermediate 9728): the
    decode step captured in a CUDA graph, whose launches overlap as programmatic dependents, must give bit
    for bit the logits of the same kernels launched one after the other; and stay within bfloat16 rounding
    of the separate-kernel path, measured against the 32-bit engine on the same weights.  Eight sequences
    take the fused products; twelve take the library products with the one-launch attention between them."""
    from dryft_b200.config import preset
    from dryft_b200.engine.api import Engine

    raw = dict(preset("qwen3-4b"))
    raw.update(num_hidden_layers=2, vocab_size=8192, max_position_embeddings=2048)
    kw = dict(seed=4, std=0.03, max_batch=16, max_seq_len=1024, max_tokens=16 * 1024)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 8192, (n,), generator=g).tolist() for n in (70, 3, 129, 64, 200, 17, 31, 90, 5, 250, 33, 128)[:n_seqs]]

    def decode_logits(**opts):
        eng = Engine.from_config(raw, **kw, **opts)
        outs = []
        with torch.inference_mode():
            s = eng.cache.open_sequences(len(prompts))
            lg = eng.stepper.step(s, prompts, [[len(p) - 1] for p in prompts])
            idx = torch.tensor(s, device="cuda")
            eng.cache.last_token[idx] = lg.argmax(-1).int()
            for _ in range(6):
                lg = eng.stepper.decode_from_state(s)[: len(prompts)].float()
                outs.append(lg.cpu())
                # the same next tokens for every engine, so that later steps stay comparable
                eng.cache.last_token[idx] = (torch.arange(len(prompts), device="cuda") * 37 + len(outs) * 11).int() % 8192
            eng.cache.close_sequences(s)
        del eng
        torch.cuda.empty_cache()
        return torch.stack(outs)

    overlapped = decode_logits(dtype="bfloat16")
    eager = decode_logits(dtype="bfloat16", cuda_graphs=False)
    in_turn = decode_logits(dtype="bfloat16", pdl=False)
    assert torch.equal(overlapped, in_turn) and torch.equal(overlapped, eager)
    separate = decode_logits(dtype="bfloat16", fuse_decode=False)
    exact = decode_logits(dtype="float32")
    tol = H.bf16_tol(separate, exact)
    assert H.rel_err(overlapped, separate) <= tol and H.rel_err(overlapped, exact) <= tol


@pytest.mark.gpu
def test_same_requests_give_the_same_logits_every_time_at_production_widths():
    """One engine, the same twelve prompts prefilled and decoded twenty times over (slots and pages are
    given back and taken again in between, L2 flushed every other time): prompt logits and decode logits
    must be the same bits every time.  Nothing may depend on when a copy, a product or a launch finishes."""
    from dryft_b200.config import preset
    from dryft_b200.engine.api import Engine

    raw = dict(preset("qwen3-4b"))
    raw.update(num_hidden_layers=2, vocab_size=8192, max_position_embeddings=2048)
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(0, 8192, (n,), generator=g).tolist() for n in (70, 3, 129, 64, 200, 17, 31, 90, 5, 250, 33, 128)]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for n_seqs in (8, 12):   # the fused decode products; the library products with the one-launch attention
        eng = Engine.from_config(raw, seed=4, std=0.03, dtype="bfloat16", max_batch=16, max_seq_len=1024, max_tokens=16 * 1024)
        first = None
        for rep in range(20):
            if rep % 2:
                flush.fill_(rep)
            outs = []
            with torch.inference_mode():
                s = eng.cache.open_sequences(n_seqs)
                lg = eng.stepper.step(s, prompts[:n_seqs], [[len(p) - 1] for p in prompts[:n_seqs]])
                outs.append(lg.float().cpu())
                idx = torch.tensor(s, device="cuda")
                eng.cache.last_token[idx] = lg.argmax(-1).int()
                for _ in range(4):
                    lg = eng.stepper.decode_from_state(s)[:n_seqs].float()
                    outs.append(lg.cpu())
                    eng.cache.last_token[idx] = lg.argmax(-1).int()
                eng.cache.close_sequences(s)
            got = torch.stack(outs)
            if first is None:
                first = got
            else:
                assert torch.equal(got, first), f"{n_seqs} sequences, repetition {rep}: logits differ from the first time"
        del eng
        torch.cuda.empty_cache()
    from dryft_b200.ops import kernels as K
    K.check_error_flags()
