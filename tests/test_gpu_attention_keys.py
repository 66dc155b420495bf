"""Tests of the bfloat16 attention kernels that one wrong key cannot pass.

With random queries and keys every key has about the same weight, so a key dropped at a page edge, a
window off by one or a stale row read from a reused page moves the output by 1/n of a value: less than
bfloat16 noise.  Here one key is made to dominate (query and key point the same way and are long, so its
score stands 50 or more above the rest): the output must be that key's value, to a bfloat16 ulp, wherever
the key lies -- position 0, the ends of a 16-key slice and of a page, the first key of a split, the last
cached key, the new token itself, the first key inside a window -- and must NOT be that value when the key
lies one place outside the window.  Freed pages are filled with NaN before they are used again: nothing of
a page's last holder may reach the next one.
"""

import math

import pytest
import torch

import helpers as H
import plain_qwen3 as P
from test_gpu_kernels import DEV, K, _attn_ref, _fill_cache

pytestmark = pytest.mark.gpu

BF = torch.bfloat16
ULP = 2.0 ** -8      # one bfloat16 rounding of the output, relative
BIG = 30.0


def _unit(d, g):
    v = torch.randn(d, generator=g)
    return v / v.norm()


def _i32(v):
    return torch.tensor(v, dtype=torch.int32, device=DEV)


# ----------------------------------------------------------------------------- decode attention
@pytest.mark.parametrize("n_heads,n_kv,d", [(8, 2, 128), (4, 2, 64), (6, 2, 48), (16, 1, 32)])
@pytest.mark.parametrize("window", [None, 100, 64, 17])
def test_attn_decode_planted_key(n_heads, n_kv, d, window):
    """Every row is a sequence of its own with 700 cached tokens and one planted key; all rows go through one
    launch, for every way of splitting (one block; clusters of 2, 3 and 8; 5 and 12 splits through memory) and
    every block shape (8, 4, 2 warps)."""
    k = K()
    page, L = 64, 700                   # cached tokens; the new token sits at position L
    scale = 1.0 / math.sqrt(d)
    g = torch.Generator().manual_seed(d + (window or 0))
    if window is None:
        # slice ends, page ends, first pages of splits (12 splits of 11 pages: one page each), last cached, own
        targets = [0, 15, 16, 63, 64, 127, 128, 333, 383, 384, 639, 640, L - 1, L]
        seen = [True] * len(targets)
    else:
        first = L - window + 1          # first visible key of the query at position L
        targets = [first, first - 1, first + 1, L - 1, L, 0]
        seen = [True, False, True, True, True, False]
    n = len(targets)
    direction = [_unit(d, g) for _ in range(n)]
    seqs, qkv_rows, want = {}, [], []
    for i, tgt in enumerate(targets):
        kseq = torch.randn(L + 1, n_kv, d, generator=g) * 0.1
        vseq = torch.randn(L + 1, n_kv, d, generator=g)
        kseq[tgt] = direction[i] * BIG
        q = (direction[i] * BIG).repeat(n_heads, 1)                    # every query head points at the key
        # the row's q | k | v as the projection would leave them: the new token's key and value are row L's
        qkv_rows.append(torch.cat([q.reshape(-1), kseq[L].reshape(-1), vseq[L].reshape(-1)]))
        seqs[i] = (kseq.to(BF), vseq.to(BF))
        want.append(seqs[i][1][tgt].float().repeat_interleave(n_heads // n_kv, dim=0).reshape(-1))
    qkv = torch.stack(qkv_rows).to(BF)
    # reference for the rows whose planted key is out of sight: plain attention over what is visible
    qf = qkv[:, :n_heads * d].view(n, n_heads, d)
    plain = torch.stack([_attn_ref(qf[i], seqs[i][0], seqs[i][1], L, scale, window) for i in range(n)])
    old = {i: (kv[0][:L], kv[1][:L]) for i, kv in seqs.items()}
    for splits, shape, cluster in ((1, 0, True), (1, 2, True), (2, 1, True), (3, 0, True), (8, 2, True), (5, 1, False), (12, 0, False),
                                   (12, 2, False)):
        if d == 256 and shape == 0:
            continue
        kc, vc, pt = _fill_cache({i: (torch.cat([kv[0], torch.full((1, n_kv, d), float("nan")).to(BF)]),
                                      torch.cat([kv[1], torch.full((1, n_kv, d), float("nan")).to(BF)])) for i, kv in old.items()},
                                 n_kv, d, page, BF, n_pages=n * 11 + 3, max_pages=11, slots=n, scatter_seed=splits + shape)
        # whatever a page's last holder left behind the sequence's end: NaN here
        for i in range(n):
            pg = int(pt[i, L // page])
            kc[pg, :, L % page + 1:] = float("nan")
            vc[pg, :, L % page + 1:] = float("nan")
        out = torch.full((n, n_heads * d), 9.0, device=DEV, dtype=BF)
        po = torch.empty(n, n_heads, splits, d, device=DEV) if splits > 1 else None
        pm = torch.empty(n, n_heads, splits, 2, device=DEV) if splits > 1 else None
        k.attn_decode(qkv.to(DEV), None, None, None, _i32(list(range(n))), _i32([L] * n), kc, vc, pt, out, n_heads, n_kv, d, 0,
                      0.0, scale, window, splits, po, pm, shape=shape, cluster=cluster)
        got = out.cpu().float()
        assert torch.isfinite(got).all(), f"splits {splits}, shape {shape}: not finite"
        for i, tgt in enumerate(targets):
            what = f"splits {splits}, shape {shape}, cluster {cluster}, key {tgt} of {L}, window {window}"
            if seen[i]:
                torch.testing.assert_close(got[i], want[i], rtol=ULP, atol=1e-3, msg=lambda m: f"{what}: {m}")
            else:
                assert (got[i] - want[i]).abs().max() > 0.5, f"{what}: a key outside the window was seen"
                torch.testing.assert_close(got[i], plain[i], rtol=2 * ULP, atol=2e-3, msg=lambda m: f"{what}: {m}")


# ----------------------------------------------------------------------------- prefill attention
def _prefill_case(kernel, n_heads, n_kv, d, window, tile):
    """Chunks that start in the middle of a page, chunks of two tokens across a page edge and inside a page,
    a long prompt from position 0.  Every sequence has one planted key; every query of the sequence points at
    it, so each query row says whether it saw the key: rows at positions target .. target + window - 1 must
    give the key's value, rows before the key or beyond the window must give plain attention over the rest."""
    k = K()
    page = 64
    scale = 1.0 / math.sqrt(d)
    g = torch.Generator().manual_seed(d + (window or 0) + tile)
    # (slot, tokens already cached, new tokens of this step, planted key)
    plan = [(0, 0, 300, 0), (1, 100, 77, 63), (2, 100, 77, 100), (3, 63, 2, 63), (4, 190, 2, 128), (5, 0, 129, 127),
            (6, 37, 150, 64), (7, 200, 60, 199), (8, 0, 1, 0), (9, 250, 6, 255)]
    seqs, dirs = {}, {}
    for slot, old, new, tgt in plan:
        Lt = old + new
        kseq = torch.randn(Lt, n_kv, d, generator=g) * 0.1
        vseq = torch.randn(Lt, n_kv, d, generator=g)
        dirs[slot] = _unit(d, g)
        kseq[tgt] = dirs[slot] * BIG
        seqs[slot] = (kseq.to(BF), vseq.to(BF))
    kc, vc, pt = _fill_cache(seqs, n_kv, d, page, BF, n_pages=40, max_pages=5, slots=10, scatter_seed=7 + tile)
    # rows of every sequence's last page behind its end hold a former holder's NaN; the step's own write of the
    # value rows clears them (zero_tail), the keys stay and must be masked
    for slot, old, new, _ in plan:
        Lt = old + new
        if Lt % page:
            pg = int(pt[slot, (Lt - 1) // page])
            kc[pg, :, Lt % page:] = float("nan")
            vc[pg, :, Lt % page:] = 0.0
    tok_slot, tok_pos, tiles0, tilesn, qs, refs, sees, wants = [], [], [], [], [], [], [], []
    base = 0
    for slot, old, new, tgt in plan:
        q = (dirs[slot] * BIG).repeat(new, n_heads, 1) + torch.randn(new, n_heads, d, generator=g) * 0.05
        q = q.to(BF)
        qs.append(q)
        for i in range(new):
            p = old + i
            tok_slot.append(slot)
            tok_pos.append(p)
            refs.append(_attn_ref(q[i], seqs[slot][0], seqs[slot][1], p, scale, window))
            sees.append(tgt <= p and (window is None or p - tgt < window))
            wants.append(seqs[slot][1][tgt].float().repeat_interleave(n_heads // n_kv, dim=0).reshape(-1))
        for q0 in range(0, new, tile):
            tiles0.append(base + q0)
            tilesn.append(min(tile, new - q0))
        base += new
    out = torch.full((base, n_heads * d), 9.0, device=DEV, dtype=BF)
    kernel(k)(torch.cat(qs).to(DEV), kc, vc, pt, _i32(tiles0), _i32(tilesn), _i32(tok_slot), _i32(tok_pos), out,
              len(tiles0), scale, window)
    torch.cuda.synchronize()
    k.check_error_flags()
    got = out.cpu().float()
    assert torch.isfinite(got).all()
    sees = torch.tensor(sees)
    assert int(sees.sum()) > 100 and int((~sees).sum()) > 20
    ref = torch.stack(refs)
    want = torch.stack(wants)
    # rows that see the key: its value to an ulp.  (The plain result is the same to 1e-6: the score gap is > 50.)
    torch.testing.assert_close(got[sees], want[sees], rtol=ULP, atol=1e-3)
    # rows that do not: nowhere near that value, and plain attention over what they do see
    assert ((got[~sees] - want[~sees]).abs().amax(dim=-1) > 0.5).all(), "a key that is out of sight was seen"
    torch.testing.assert_close(got[~sees], ref[~sees], rtol=2 * ULP, atol=3e-3)


@pytest.mark.parametrize("n_heads,n_kv,d", [(8, 2, 128), (6, 2, 48), (3, 3, 64)])
@pytest.mark.parametrize("window", [None, 40, 64, 65])
def test_attn_prefill_planted_key(n_heads, n_kv, d, window):
    _prefill_case(lambda k: k.attn_prefill, n_heads, n_kv, d, window, tile=64)


@pytest.mark.parametrize("n_heads,n_kv,d", [(8, 2, 128), (4, 1, 128), (3, 3, 64)])
@pytest.mark.parametrize("window", [None, 40, 64, 65, 129])
def test_attn_prefill_tc_planted_key(n_heads, n_kv, d, window):
    _prefill_case(lambda k: k.attn_prefill_tc, n_heads, n_kv, d, window, tile=128)


# ----------------------------------------------------------------------------- cache write with tail zeroing
@pytest.mark.parametrize("d,n_kv", [(128, 2), (48, 3), (20, 1)])
def test_value_rows_behind_a_sequences_last_token_are_zeroed(d, n_kv):
    """``qk_norm_rope_store(zero_tail=True)``: the last token each sequence brings clears the value rows of its
    page behind its own row, and nothing else: keys, other pages, other sequences' rows stay as they were."""
    k = K()
    n_heads, page = 2 * n_kv, 64
    rot = d if d % 4 == 0 and d != 20 else 0
    # three sequences: 5 tokens from 60 (crosses into a second page), 1 token at 63 (last row: no tail), 3 from 0
    plan = [(0, 60, 5), (2, 63, 1), (1, 0, 3)]
    tok_slot = sum(([s] * n for s, _, n in plan), []) + [-1]
    tok_pos = sum((list(range(o, o + n)) for _, o, n in plan), []) + [0]
    n = len(tok_slot)
    pt = _i32([[3, 5], [1, 0], [4, 2]])
    kc = torch.full((6, n_kv, page, d), 7.0, device=DEV, dtype=BF)
    vc = torch.full((6, n_kv, page, d), 7.0, device=DEV, dtype=BF)
    qkv = torch.randn(n, (n_heads + 2 * n_kv) * d).to(BF).to(DEV)
    q_out = torch.empty(n, n_heads, d, device=DEV, dtype=BF)
    inv_freq = (1.0 / (1e4 ** (torch.arange(0, rot, 2).float() / rot))).to(DEV) if rot else None
    for use_table in (False, True):
        kc.fill_(7.0); vc.fill_(7.0)
        table = k.rope_table(_i32(tok_pos), inv_freq, n, BF) if (use_table and rot) else None
        k.qk_norm_rope_store(qkv, None, None, inv_freq, _i32(tok_slot), _i32(tok_pos), q_out, kc, vc, pt, n_heads, n_kv, d, rot,
                             0.0, cs_table=table, zero_tail=True)
        v = vc.cpu().float()
        written = torch.zeros(6, page, dtype=torch.bool)
        zeroed = torch.zeros(6, page, dtype=torch.bool)
        for (slot, old, new), pages in zip(plan, ([3, 5], [4, 2], [1, 0])):
            for p in range(old, old + new):
                written[pages[p // page], p % page] = True
            last = old + new - 1
            zeroed[pages[last // page], last % page + 1:] = True
        for pg in range(6):
            for r in range(page):
                row = v[pg, :, r]
                if zeroed[pg, r]:
                    assert (row == 0).all(), f"page {pg} row {r} should be zero"
                elif not written[pg, r]:
                    assert (row == 7.0).all(), f"page {pg} row {r} was touched"
        kk = kc.cpu().float()
        assert ((kk == 7.0).all(dim=-1).all(dim=1) == ~written).all(), "keys: exactly the written rows change"


# ----------------------------------------------------------------------------- whole model on poisoned pages
@pytest.mark.parametrize("name", ["b", "d"])
def test_freed_pages_full_of_nan_do_not_reach_the_next_request(model_dirs, name):
    """Every page of the cache is filled with NaN while no sequence is live (what a request that overflowed
    would leave behind); the next requests -- prompts, then tokens one by one, alone and in a batch -- must
    still match the plain implementation."""
    from dryft_b200.engine.api import Engine

    eng = Engine(model_dirs[name], dtype="bfloat16", max_batch=4, max_seq_len=512, max_tokens=4 * 512)
    plain32 = P.load_plain(model_dirs[name], torch.float32)
    plainb = P.load_plain(model_dirs[name], BF)
    for g in eng.cache._groups:
        g.k.fill_(float("nan"))
        g.v.fill_(float("nan"))
    seqs = H.prompts_for(name, [90, 37, 140], seed=55)
    with torch.inference_mode():
        slots = eng.cache.open_sequences(3)
        heads = [70, 5, 129]
        rows = {i: [] for i in range(3)}
        out = eng.stepper.step(slots, [s[:h] for s, h in zip(seqs, heads)], [[h - 1] for h in heads])
        for i in range(3):
            rows[i].append(out[i:i + 1])
        fed = list(heads)
        alive = [0, 1, 2]
        while alive:
            out = eng.stepper.step([slots[i] for i in alive], [[seqs[i][fed[i]]] for i in alive], [[0] for _ in alive])
            for j, i in enumerate(alive):
                rows[i].append(out[j:j + 1])
                fed[i] += 1
            done = [i for i in alive if fed[i] >= len(seqs[i])]
            eng.cache.close_sequences([slots[i] for i in done])
            alive = [i for i in alive if i not in done]
    for i in range(3):
        got = torch.cat(rows[i]).float().cpu()
        assert torch.isfinite(got).all(), f"request {i}: NaN from a freed page reached the logits"
        at = list(range(heads[i] - 1, len(seqs[i])))
        p32 = plain32.logits(seqs[i])[at]
        pb = plainb.logits(seqs[i])[at]
        assert H.rel_err(got, pb) <= H.bf16_tol(pb, p32)
