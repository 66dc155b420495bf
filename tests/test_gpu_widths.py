"""The benchmark's own kernel instantiations and schedules against the plain implementation.

Two layers at the Qwen3-4B widths (hidden 2560, 32 / 8 heads of 128, intermediate 9728; vocabulary 8192),
written with ``write_random_model`` on the CPU so that ``tests/plain_qwen3.py`` loads the same tensors:
whole requests, the last 32 tokens one by one, unequal batches of 12, 16 and 64 sequences whose shorter
requests end earlier (the decode path above 8 rows), generation with CUDA graphs across a context-bucket
edge and across batch-bucket edges with stop tokens, greedy and sampled.

And the edges of the schedules themselves, on a small configuration with the widths that take the
per-inner-size decode products (cheap for the plain model): every context bucket -1 / 0 / +1, every
batch bucket and one more (the reference's ``shapes`` prompt set, ``agent/prompts.py:120-138``), one
sequence -> a big batch -> one sequence again giving the same bits (``agent/verify.py:145-154``), and a
context long enough for more than eight attention splits (partials through memory, combined by the last
block to finish).
"""

import pytest
import torch

import helpers as H
import plain_qwen3 as P

pytestmark = pytest.mark.gpu

WIDE = dict(num_hidden_layers=2, hidden_size=2560, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
            intermediate_size=9728, vocab_size=8192, rope_theta=5000000.0, rms_norm_eps=1e-6,
            tie_word_embeddings=True, max_position_embeddings=2048)
# config "d" of the tiny set with room for long contexts
LONG = dict(H.TINY["d"], max_position_embeddings=16384)
CONFIGS = {"wide": (WIDE, 11, 0.03), "long": (LONG, 12, 0.08)}
DTYPES = [torch.float32, torch.bfloat16]


def _raw(name):
    base = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_act": "silu",
            "attention_bias": False, "rope_scaling": None}
    base.update(CONFIGS[name][0])
    return base


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    from dryft_b200.weights import write_random_model

    out = {}
    for name, (_, seed, std) in CONFIGS.items():
        d = str(tmp_path_factory.mktemp(f"model_{name}"))
        write_random_model(_raw(name), seed, d, std=std)
        out[name] = d
    return out


_engines, _plains, _logits = {}, {}, {}


def engine(dirs, name, dtype, **kw):
    from dryft_b200.engine.api import Engine

    key = (name, dtype, tuple(sorted(kw.items())))
    if key not in _engines:
        _engines[key] = Engine(dirs[name], dtype=dtype, **kw)
    return _engines[key]


def plain_logits(dirs, name, dtype, tokens):
    """Plain logits of the whole sequence, remembered (the bfloat16 checks need both precisions)."""
    key = (name, dtype, tuple(tokens))
    if key not in _logits:
        if (name, dtype) not in _plains:
            _plains[(name, dtype)] = P.load_plain(dirs[name], dtype)
        _logits[key] = _plains[(name, dtype)].logits(list(tokens))
    return _logits[key]


def prompts(name, lengths, seed):
    g = torch.Generator().manual_seed(4000 + seed)
    vocab = CONFIGS[name][0]["vocab_size"]
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]


def check(got, dirs, name, dtype, tokens, rows, what):
    got = got.float().cpu()
    assert torch.isfinite(got).all(), what
    p32 = plain_logits(dirs, name, torch.float32, tokens)[rows]
    if dtype == torch.float32:
        e = H.rel_err(got, p32)
        assert e <= H.FP32_TOL, f"{what}: 32-bit logits off by {e:.3g}"
    else:
        pb = plain_logits(dirs, name, torch.bfloat16, tokens)[rows]
        tol = H.bf16_tol(pb, p32)
        e = H.rel_err(got, pb)
        assert e <= tol, f"{what}: bfloat16 logits off by {e:.3g} (allowed {tol:.3g})"


def step(eng, slots, tokens, want):
    with torch.inference_mode():
        return eng.stepper.step(slots, tokens, want)


def same_choices(dirs, name, dtype, prompt, one, other, what):
    """Two runs of one sequence in different company.  32-bit: the same tokens.  bfloat16: the company decides
    which kernels run (library products above 16 rows, register-streaming ones below), whose sums round
    differently, so the runs agree up to the first position where the plain model's logits of the two choices
    lie closer together than bfloat16 rounding moves them; from there each run is checked on its own."""
    if list(one) == list(other):
        return
    assert dtype == torch.bfloat16, what
    i = next(j for j in range(min(len(one), len(other))) if one[j] != other[j])
    seq_tokens = list(prompt) + list(one[:i])
    lg = plain_logits(dirs, name, torch.float32, seq_tokens)[-1]
    pb = plain_logits(dirs, name, torch.bfloat16, seq_tokens)[-1]
    allowed = 2.0 * float((pb - lg).abs().max()) + 1e-3 * float(lg.abs().max())
    gap = abs(float(lg[one[i]] - lg[other[i]]))
    assert gap <= allowed, f"{what}: token {i} is {one[i]} / {other[i]}, plain logits {gap:.3g} apart (allowed {allowed:.3g})"


def check_generated(dirs, name, dtype, prompt, ours, what, temperature=0.0, top_k=0, seed=0, seq=0):
    """Teacher-forced check of generated tokens (``agent/verify.py:100-109``): one plain pass over the prompt and
    our tokens.  32-bit: every token is the plain model's choice (argmax, or the same draw).  bfloat16, greedy:
    our token's plain logit is within what bfloat16 rounding does to these logits of the best one."""
    seq_tokens = list(prompt) + list(ours[:-1])
    lg = plain_logits(dirs, name, torch.float32, seq_tokens)[len(prompt) - 1:]
    assert lg.shape[0] == len(ours)
    if dtype == torch.float32:
        for t, tok in enumerate(ours):
            want = P.choose_token(lg[t], temperature, top_k, P.uniform_draw(seed, seq, t))
            if want != tok:   # a choice may only differ at an exact near-tie of the 32-bit logits
                gap = abs(float(lg[t][want] - lg[t][tok]))
                assert temperature == 0.0 and gap <= 2 * H.FP32_TOL * float(lg[t].abs().max()), \
                    f"{what}: token {t} is {tok}, plain chooses {want}"
    else:
        pb = plain_logits(dirs, name, torch.bfloat16, seq_tokens)[len(prompt) - 1:]
        allowed = 2.0 * float((pb - lg).abs().max()) + 1e-3 * float(lg.abs().max())
        best = lg.max(dim=-1).values
        mine = lg.gather(1, torch.tensor(ours)[:, None])[:, 0]
        m = float((best - mine).max())
        assert m <= allowed, f"{what}: teacher-forced margin {m:.3g} (allowed {allowed:.3g})"


# ----------------------------------------------------------------------------- 4B widths: logits
@pytest.mark.parametrize("dtype", DTYPES)
def test_wide_whole_and_last_32_one_by_one(dirs, dtype):
    eng = engine(dirs, "wide", dtype, max_batch=64, max_seq_len=1280, max_tokens=64 * 128 + 2048)
    for i, n in enumerate([1, 129, 200]):
        toks = prompts("wide", [n], i)[0]
        (slot,) = eng.cache.open_sequences(1)
        got = step(eng, [slot], [toks], [list(range(n))])
        eng.cache.close_sequences([slot])
        check(got, dirs, "wide", dtype, toks, list(range(n)), f"wide whole len {n}")
    toks = prompts("wide", [100], 7)[0]
    (slot,) = eng.cache.open_sequences(1)
    rows = [step(eng, [slot], [toks[:68]], [[67]])]
    for t in toks[68:]:
        rows.append(step(eng, [slot], [[t]], [[0]]))
    eng.cache.close_sequences([slot])
    check(torch.cat(rows), dirs, "wide", dtype, toks, list(range(67, 100)), "wide last 32 one by one")
    eng.cache.check()


@pytest.mark.parametrize("dtype,stream", [(torch.float32, 0), (torch.bfloat16, 0), (torch.bfloat16, 64)])
def test_wide_unequal_batches_of_12_16_64(dirs, dtype, stream):
    """Above eight rows the decode step changes kernels (library products, separate norm and SiLU*mul launches,
    narrower attention blocks; or, with ``stream_m_max=64``, the tcgen05 weight-streaming products with the norm,
    the residual add and SiLU*mul fused in); as sequences end the batch shrinks through 8 rows into the
    register-streaming products.  Three batches in a row on the same slots."""
    kw = dict(stream_m_max=stream) if stream else {}
    eng = engine(dirs, "wide", dtype, max_batch=64, max_seq_len=1280, max_tokens=64 * 128 + 2048, **kw)
    g = torch.Generator().manual_seed(77)
    seed = 100
    for n_seqs in (12, 16, 64):
        plens = torch.randint(1, 41, (n_seqs,), generator=g).tolist()
        extra = torch.randint(0, 8, (n_seqs,), generator=g).tolist()
        extra[0], extra[1] = 0, 10          # one ends right after its prompt, one lasts longest
        batch = list(zip(plens, [p + e for p, e in zip(plens, extra)]))
        seqs = []
        for (_, tl) in batch:
            seed += 1
            seqs.append(prompts("wide", [tl], seed)[0])
        slots = eng.cache.open_sequences(n_seqs)
        got = {i: [] for i in range(n_seqs)}
        rows_of = {i: [] for i in range(n_seqs)}
        out = step(eng, slots, [s[:pl] for s, (pl, _) in zip(seqs, batch)], [[pl - 1] for (pl, _) in batch])
        for i, (pl, _) in enumerate(batch):
            got[i].append(out[i:i + 1])
            rows_of[i].append(pl - 1)
        fed = [pl for (pl, _) in batch]
        alive = [i for i, (pl, tl) in enumerate(batch) if pl < tl]
        eng.cache.close_sequences([slots[i] for i in range(n_seqs) if i not in alive])
        sizes = set()
        while alive:
            sizes.add(len(alive))
            out = step(eng, [slots[i] for i in alive], [[seqs[i][fed[i]]] for i in alive], [[0] for _ in alive])
            for j, i in enumerate(alive):
                got[i].append(out[j:j + 1])
                rows_of[i].append(fed[i])
                fed[i] += 1
            done = [i for i in alive if fed[i] >= batch[i][1]]
            eng.cache.close_sequences([slots[i] for i in done])
            alive = [i for i in alive if i not in done]
        assert max(sizes) > 8 and min(sizes) <= 8, "the batch must shrink across the 8-row edge"
        for i in range(n_seqs):
            check(torch.cat(got[i]), dirs, "wide", dtype, seqs[i], rows_of[i], f"wide batch of {n_seqs}, request {i}")
        eng.cache.check()
    assert eng.cache.slots.n_held == 0


# ----------------------------------------------------------------------------- 4B widths: generation with graphs
@pytest.mark.parametrize("dtype", DTYPES)
def test_wide_generation_across_the_1024_context_edge(dirs, dtype):
    """A 1,000-token prompt and 40 new tokens: the context crosses 1,024 keys mid-generation, so a second graph
    (another split of the keys) is captured with a step in flight; a short second sequence rides along."""
    eng = engine(dirs, "wide", dtype, max_batch=64, max_seq_len=1280, max_tokens=64 * 128 + 2048)
    ps = prompts("wide", [1000, 9], 31)
    out = [s for s in eng.generate(ps, 40)]
    assert len(out) == 40
    assert [s for s in eng.generate(ps, 40)] == out, "second run differs from the first"
    for b, p in enumerate(ps):
        check_generated(dirs, "wide", dtype, p, [s[b] for s in out], f"wide across 1024, sequence {b}")
    if dtype == torch.float32:
        out = [s for s in eng.generate(ps[:1], 30, temperature=0.8, top_k=50, seed=5)]
        check_generated(dirs, "wide", dtype, ps[0], [s[0] for s in out], "wide across 1024, sampled", 0.8, 50, 5, 0)
    from dryft_b200.ops import kernels as K
    K.check_error_flags()
    assert eng.cache.slots.n_held == 0


def test_wide_generation_with_the_streaming_products_equals_their_step_by_step_run(dirs):
    """``stream_m_max=64``: seventeen sequences decoded through the captured graph (programmatic launches, tickets
    and workspace shared by all layers) must give the tokens of the plain model, twice over."""
    eng = engine(dirs, "wide", torch.bfloat16, max_batch=64, max_seq_len=1280, max_tokens=64 * 128 + 2048, stream_m_max=64)
    ps = prompts("wide", [3, 17, 8, 30, 1, 12, 25, 6, 9, 14, 2, 21, 5, 11, 7, 19, 4], 43)
    out = [s for s in eng.generate(ps, 10)]
    assert [s for s in eng.generate(ps, 10)] == out
    for b, p in enumerate(ps):
        check_generated(dirs, "wide", torch.bfloat16, p, [s[b] for s in out], f"streaming products, sequence {b}")
    from dryft_b200.ops import kernels as K
    K.check_error_flags()
    assert int(K.gemm_stream_scratch(eng.device)[1].abs().sum()) == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sampled", [False, True])
def test_wide_generation_across_batch_bucket_edges_with_stop_tokens(dirs, dtype, sampled):
    """Seventeen sequences (bucket 24) that stop tokens take out one after another: the padded batch goes
    24 -> 16 -> 8 -> 4 ... while it runs, from the library products into the fused ones."""
    if sampled and dtype == torch.bfloat16:
        pytest.skip("a sampled draw is only comparable in 32-bit")
    eng = engine(dirs, "wide", dtype, max_batch=64, max_seq_len=1280, max_tokens=64 * 128 + 2048)
    ps = prompts("wide", [3, 17, 8, 30, 1, 12, 25, 6, 9, 14, 2, 21, 5, 11, 7, 19, 4], 41)
    kw = dict(temperature=0.7, top_k=20, seed=3) if sampled else {}
    free = [s for s in eng.generate(ps, 14, **kw)]
    # stop tokens taken from the free run so that sequences leave at steps 2, 4, 5, 7, 9 and 11
    stops = sorted({free[2][0], free[4][5], free[5][9], free[7][12], free[9][3], free[11][16]})
    got = [s for s in eng.generate(ps, 14, stop_token_ids=stops, **kw)]
    alive_counts = [sum(t != -1 for t in s) for s in got]
    assert alive_counts[0] == 17 and min(alive_counts) < 17
    for b, p in enumerate(ps):
        col = [s[b] for s in got]
        n = next((i + 1 for i, t in enumerate(col) if t in stops), len(col))
        assert all(t == -1 for t in col[n:]) and all(t >= 0 for t in col[:n]), f"sequence {b}: {col}"
        # a sequence's tokens do not depend on who else is still in the batch: equal to the free run's
        same_choices(dirs, "wide", dtype, p, col[:n], [s[b] for s in free][:n], f"sequence {b} changed when others left")
        check_generated(dirs, "wide", dtype, p, col[:n], f"wide stops, sequence {b}", seq=b, **kw)
    many = eng.generate_many(ps, 14, stop_token_ids=stops, **kw)
    for b in range(len(ps)):
        col = [s[b] for s in got]
        assert many[b] == [t for t in col if t != -1]
    eng.cache.check()
    assert eng.cache.slots.n_held == 0


def test_wide_one_sequence_then_a_big_batch_then_one_again_same_bits(dirs):
    """b1 -> big batch -> b1 (``agent/verify.py:145-154``): nothing a big batch leaves behind (graphs, pages,
    state, scratch) may change a later small one.  Tokens and prompt logits, bit for bit, in bfloat16."""
    eng = engine(dirs, "wide", torch.bfloat16, max_batch=64, max_seq_len=1280, max_tokens=64 * 128 + 2048)
    one = prompts("wide", [70], 51)
    big = prompts("wide", [5 + 3 * i for i in range(33)], 52)

    def run_one():
        toks = [s[0] for s in eng.generate(one, 12)]
        s = eng.cache.open_sequences(1)
        lg = step(eng, s, one, [[69]]).float().cpu()
        eng.cache.close_sequences(s)
        return toks, lg

    a = run_one()
    list(eng.generate(big, 6))
    b = run_one()
    assert a[0] == b[0] and torch.equal(a[1], b[1])


# ----------------------------------------------------------------------------- schedule edges, small widths
@pytest.mark.parametrize("dtype", DTYPES)
def test_every_context_bucket_edge(dirs, dtype):
    """Contexts that end just below, on and just above 1,024 and 2,048 keys (the graph's context bucket is
    chosen from the longest sequence plus one), each with a short companion, four new tokens."""
    eng = engine(dirs, "long", dtype, max_batch=24, max_seq_len=9000, max_tokens=9000 + 23 * 256)
    for edge in (1024, 2048):
        for n in (edge - 3, edge - 2, edge - 1, edge, edge + 1):
            ps = prompts("long", [n, 3], n)
            out = [s for s in eng.generate(ps, 4)]
            for b, p in enumerate(ps):
                check_generated(dirs, "long", dtype, p, [s[b] for s in out], f"context edge: prompt {n}, sequence {b}")
    assert eng.cache.slots.n_held == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_every_batch_bucket_and_one_more(dirs, dtype):
    eng = engine(dirs, "long", dtype, max_batch=24, max_seq_len=9000, max_tokens=9000 + 23 * 256)
    for n_seqs in (1, 2, 3, 4, 5, 8, 9, 16, 17, 24):
        ps = prompts("long", [1 + (5 * i + n_seqs) % 23 for i in range(n_seqs)], 60 + n_seqs)
        out = [s for s in eng.generate(ps, 5)]
        assert len(out) == 5 and all(len(s) == n_seqs for s in out)
        for b, p in enumerate(ps):
            check_generated(dirs, "long", dtype, p, [s[b] for s in out], f"batch of {n_seqs}, sequence {b}")
    assert eng.cache.slots.n_held == 0


def test_small_batch_is_unchanged_by_a_big_one_between(dirs):
    eng = engine(dirs, "long", torch.bfloat16, max_batch=24, max_seq_len=9000, max_tokens=9000 + 23 * 256)
    one = prompts("long", [40], 71)
    big = prompts("long", [2 + i for i in range(24)], 72)
    a = [s[0] for s in eng.generate(one, 20)]
    list(eng.generate(big, 8))
    assert [s[0] for s in eng.generate(one, 20)] == a


@pytest.mark.parametrize("dtype", DTYPES)
def test_more_than_eight_attention_splits(dirs, dtype):
    """Beyond 8,192 keys the decode attention splits a sequence's keys over more blocks than a cluster holds:
    the partial results meet in memory and the last block to finish combines them.  One sequence of 8,200 tokens,
    then four tokens one by one through the step function, and the same four through the captured graph."""
    eng = engine(dirs, "long", dtype, max_batch=24, max_seq_len=9000, max_tokens=9000 + 23 * 256)
    n = 8200
    toks = prompts("long", [n + 4], 81)[0]
    (slot,) = eng.cache.open_sequences(1)
    rows = [step(eng, [slot], [toks[:n]], [[n - 1]])]
    for t in toks[n:]:
        rows.append(step(eng, [slot], [[t]], [[0]]))
    eng.cache.close_sequences([slot])
    check(torch.cat(rows), dirs, "long", dtype, toks, list(range(n - 1, n + 4)), "8,200 keys, token by token")
    # the same tokens through the captured decode graph, fed from the per-sequence state
    (slot,) = eng.cache.open_sequences(1)
    rows = [step(eng, [slot], [toks[:n]], [[n - 1]])]
    with torch.inference_mode():
        for t in toks[n:]:
            eng.cache.last_token[slot] = t
            rows.append(eng.stepper.decode_from_state([slot])[:1].clone())
    eng.cache.close_sequences([slot])
    check(torch.cat(rows), dirs, "long", dtype, toks, list(range(n - 1, n + 4)), "8,200 keys, captured graph")
    from dryft_b200.ops import kernels as K
    K.check_error_flags()


@pytest.mark.parametrize("dtype", DTYPES)
def test_prompt_steps_replayed_from_a_captured_graph(dirs, dtype):
    """A prompt step's launches depend only on (tokens, sequences, wanted rows, tiles): the second step of a shape is
    captured, later ones are replayed with other tokens, other lengths (300 + 100, then 110 + 290: the same counts),
    other slots and other starting positions (a chunk continuing a sequence).  Every result is compared with the
    plain implementation; results handed out earlier must not change when the graph runs again."""
    eng = engine(dirs, "long", dtype, max_batch=24, max_seq_len=9000, max_tokens=9000 + 23 * 256)
    assert eng.stepper.cuda_graphs
    kept = []
    cases = [(300, 100), (300, 100), (110, 290), (256, 144), (300, 100)]
    for i, (a, b) in enumerate(cases):
        ps = prompts("long", [a, b], 90 + i)
        slots = eng.cache.open_sequences(2 + i % 2)[-2:]          # other slots from one step to the next
        got = step(eng, slots, ps, [[a - 1, 0], [b - 1]])
        kept.append((got, got.clone(), ps))
        eng.cache.close_sequences([s for s in range(eng.cache.max_slots) if eng.cache.slots.is_held(s)])
        check(got[:2], dirs, "long", dtype, ps[0], [a - 1, 0], f"prompt graph, case {i}, first sequence")
        check(got[2:], dirs, "long", dtype, ps[1], [b - 1], f"prompt graph, case {i}, second sequence")
    tile = eng.stepper.prefill_tile
    assert (400, 2, 3, -(-300 // tile) + -(-100 // tile)) in eng.stepper._prompt_graphs
    for got, copy, _ in kept:
        assert torch.equal(got, copy), "a later replay changed logits handed out earlier"
    # a chunk that continues two sequences (positions 64.. and 10..): again 400 tokens, 2 sequences, 3 rows, 4 tiles
    ps = prompts("long", [64 + 300, 10 + 100], 99)
    slots = eng.cache.open_sequences(2)
    step(eng, slots, [ps[0][:64], ps[1][:10]], [[], []])
    got = step(eng, slots, [ps[0][64:], ps[1][10:]], [[299, 0], [99]])
    eng.cache.close_sequences(slots)
    check(got[:2], dirs, "long", dtype, ps[0], [363, 64], "prompt graph, continued chunk, first sequence")
    check(got[2:], dirs, "long", dtype, ps[1], [109], "prompt graph, continued chunk, second sequence")
    eng.cache.check()
    assert eng.cache.slots.n_held == 0
