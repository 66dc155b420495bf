"""The plain implementation itself: closed-form cases of each part, structural properties (causality,
window), its two precisions, its token choice — and, once, its agreement with hari495/dryft's own
model code on tiny random models (``tests/golden``)."""

import math
import os
import sys

import pytest
import torch
from safetensors.torch import load_file

import plain_qwen3 as P

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
from golden_weights import CASES, make_weights  # noqa: E402

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_rmsnorm_closed_form():
    x = torch.tensor([[3.0, 4.0]])
    w = torch.tensor([2.0, 0.5])
    # mean square = 12.5; eps 0 -> x / sqrt(12.5)
    y = P.rmsnorm(x, w, 0.0)
    torch.testing.assert_close(y, torch.tensor([[2 * 3 / math.sqrt(12.5), 0.5 * 4 / math.sqrt(12.5)]]))
    # bf16: the normalised value is rounded BEFORE the weight multiplies
    xb = torch.tensor([[1.0, 2.0, 3.0, 5.0]], dtype=torch.bfloat16)
    wb = torch.tensor([1.5, 1.25, 0.75, 1.125], dtype=torch.bfloat16)
    xf = xb.float()
    n = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6)).to(torch.bfloat16)
    assert torch.equal(P.rmsnorm(xb, wb, 1e-6), (wb.float() * n.float()).to(torch.bfloat16))


def test_rope_rotates_pairs_and_keeps_norm():
    D = 8
    x = torch.randn(5, 2, D)
    cos, sin = P.rope_cos_sin(torch.arange(5), D, 10000.0, torch.float32)
    y = P.apply_rope(x, cos, sin)
    assert torch.equal(y[0], x[0])  # position 0: no rotation
    torch.testing.assert_close(y.norm(dim=-1), x.norm(dim=-1))
    # dims j and j + D/2 rotate together by pos * theta^(-2j/D)
    j, pos = 1, 3
    ang = pos * 10000.0 ** (-2 * j / D)
    a, b = x[pos, 0, j], x[pos, 0, j + D // 2]
    torch.testing.assert_close(y[pos, 0, j], a * math.cos(ang) - b * math.sin(ang))
    torch.testing.assert_close(y[pos, 0, j + D // 2], b * math.cos(ang) + a * math.sin(ang))
    assert torch.equal(P.rotate_half(torch.tensor([1.0, 2.0, 3.0, 4.0])), torch.tensor([-3.0, -4.0, 1.0, 2.0]))


def test_attention_is_causal_grouped_and_windowed():
    T, nH, nKV, D = 6, 4, 2, 8
    q, k, v = torch.randn(T, nH, D), torch.randn(T, nKV, D), torch.randn(T, nKV, D)
    o = P.causal_attention(q, k, v, 0.3, None, torch.float32).view(T, nH, D)
    torch.testing.assert_close(o[0, 0], v[0, 0])  # the first token sees only itself
    torch.testing.assert_close(o[0, 3], v[0, 1])  # q head 3 reads kv head 3 // 2 = 1
    # by hand for the last token, head 2 (kv head 1)
    s = (k[:, 1] @ q[5, 2]) * 0.3
    torch.testing.assert_close(o[5, 2], torch.softmax(s, 0) @ v[:, 1])
    # changing a later key/value leaves earlier outputs alone
    k2, v2 = k.clone(), v.clone()
    k2[4:] += 1.0
    v2[4:] -= 1.0
    o2 = P.causal_attention(q, k2, v2, 0.3, None, torch.float32).view(T, nH, D)
    assert torch.equal(o2[:4], o[:4]) and not torch.equal(o2[4:], o[4:])
    # window 2: token 5 sees keys 4 and 5 only
    ow = P.causal_attention(q, k, v, 0.3, 2, torch.float32).view(T, nH, D)
    s = (k[4:6, 0] @ q[5, 0]) * 0.3
    torch.testing.assert_close(ow[5, 0], torch.softmax(s, 0) @ v[4:6, 0])
    torch.testing.assert_close(ow[1], o[1])  # positions inside the window are unchanged


def test_silu_mul_and_matmul_rounding():
    g = torch.tensor([0.0, 1.0, -2.0])
    u = torch.tensor([5.0, 2.0, 3.0])
    torch.testing.assert_close(P.silu_mul(g, u), torch.tensor([0.0, 2 / (1 + math.exp(-1)), -6 / (1 + math.exp(2))]))
    gb = torch.tensor([1.3], dtype=torch.bfloat16)
    ub = torch.tensor([2.7], dtype=torch.bfloat16)
    s = (gb.float() / (1 + torch.exp(-gb.float()))).to(torch.bfloat16)
    assert torch.equal(P.silu_mul(gb, ub), (s.float() * ub.float()).to(torch.bfloat16))
    x = torch.randn(3, 5).to(torch.bfloat16)
    w = torch.randn(4, 5).to(torch.bfloat16)
    assert torch.equal(P.matmul_nt(x, w, torch.bfloat16), (x.float() @ w.float().T).to(torch.bfloat16))


def _plain_case(name, dtype):
    case = CASES[name]
    w = make_weights(case["config"], case["seed"], case["std"])
    if dtype == torch.bfloat16:
        w = {k: v.to(torch.bfloat16) for k, v in w.items()}
    return case, P.PlainQwen3(case["config"], w, dtype)


def test_model_is_causal_and_deterministic():
    case, m = _plain_case("tiny_b", torch.float32)
    ids = case["prompts"][3]
    a = m.logits(ids)
    b = m.logits(ids[:20])
    torch.testing.assert_close(a[:20], b, rtol=1e-5, atol=1e-6)
    assert torch.equal(m.logits(ids), a)


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
@pytest.mark.parametrize("tag,dtype", [("f32", torch.float32), ("bf16", torch.bfloat16)])
def test_plain_matches_reference_model_code(name, tag, dtype):
    """Golden logits made by ``tests/golden/make_golden.py`` from the reference's ``Model.prefill`` and
    ``Model.decode_step`` on the CPU: ragged prompts, then greedy steps.  The plain implementation,
    teacher-forced with the reference's tokens, must give the same logits at every step."""
    gold = load_file(os.path.join(GOLDEN, f"{name}_{tag}.safetensors"))
    case, m = _plain_case(name, dtype)
    toks = gold["tokens"].tolist()  # [steps][B]
    worst = 0.0
    for b, prompt in enumerate(case["prompts"]):
        full = list(prompt) + [toks[t][b] for t in range(case["steps"] - 1)]
        lg = m.logits(full)[len(prompt) - 1:]
        ref = torch.cat([gold["prefill_logits"][b:b + 1], gold["decode_logits"][:, b]])
        err = float((lg - ref).abs().max() / ref.abs().max())
        worst = max(worst, err)
        if dtype == torch.float32:
            assert [int(x) for x in lg.argmax(-1)] == [toks[t][b] for t in range(case["steps"])]
    # 32-bit: sums in another order only.  bfloat16: the reference rounds its logits to bf16
    # (model.py:186,261; 2^-9 relative to the largest logit) and its attention sums in another order.
    assert worst <= (2e-5 if dtype == torch.float32 else 2e-2), worst


def test_choose_token_properties():
    lg = torch.tensor([0.1, 3.0, 3.0, -1.0, 2.9])
    assert P.choose_token(lg, 0.0, 0, 0.5) == 1  # greedy: first index of the maximum
    # top-k 1 always gives the (first) maximum whatever the draw
    assert {P.choose_token(lg, 1.0, 1, u) for u in (0.0, 0.3, 0.999)} == {1}
    # top-k 2 with a tie at the boundary keeps the lower indices (1 and 2), never index 4
    picks = {P.choose_token(lg, 1.0, 2, u / 100) for u in range(100)}
    assert picks == {1, 2}
    # u -> 0 gives the first kept index, u -> 1 the last kept index
    assert P.choose_token(lg, 1.0, 0, 0.0) == 0 and P.choose_token(lg, 1.0, 0, 0.9999999) == 4
    # frequencies follow the softmax
    p = torch.softmax(lg / 0.7, 0)
    n = 4000
    counts = torch.zeros(5)
    for i in range(n):
        counts[P.choose_token(lg, 0.7, 0, P.uniform_draw(7, 0, i))] += 1
    assert float((counts / n - p).abs().max()) < 0.03


def test_uniform_draw_is_a_pure_function_of_its_key():
    a = P.uniform_draw(1, 2, 3)
    assert a == P.uniform_draw(1, 2, 3) and 0.0 <= a < 1.0
    assert len({P.uniform_draw(1, s, t) for s in range(20) for t in range(20)}) == 400
    xs = [P.uniform_draw(5, 0, t) for t in range(2000)]
    assert abs(sum(xs) / len(xs) - 0.5) < 0.03
