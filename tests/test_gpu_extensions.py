"""What another architecture would need, shown with toy parts defined here and registered without a change to
the library: a mixer that keeps two kinds of state at once (a short tail of past inputs and a running sum), a
norm of another arithmetic that must never be folded into the fused decode products although its class bears
the stock norm's name, prompts fed in chunks, and random weights that mean one model wherever they are drawn."""

import pytest
import torch

import helpers as H
import plain_qwen3 as P

pytestmark = pytest.mark.gpu


def _toy_arch(name, norm_kind, mixers, hidden, vocab, heads=(4, 2, 64), inter=512):
    """A config class for a toy architecture: ``mixers`` is a list of mixer kinds ("attention" or a toy kind)."""
    from dryft_b200.config.spec import LayerSpec, ModelSpec, PartSpec, RunStep

    class ToyConfig:
        def __init__(self, raw):
            self.raw = dict(raw)

        def to_dict(self):
            return dict(self.raw)

        def model_spec(self):
            nh, nkv, d = heads
            norm = PartSpec(norm_kind, {"size": hidden, "eps": 1e-5})
            attn = PartSpec("attention", {"hidden_size": hidden, "num_heads": nh, "num_kv_heads": nkv, "head_dim": d,
                                          "scale": d ** -0.5, "window": None, "qk_norm": None,
                                          "position": PartSpec("rope", {"rotary_dim": d, "theta": 1e4})})
            ffn = PartSpec("swiglu", {"hidden_size": hidden, "intermediate_size": inter})
            layers = tuple(LayerSpec("prenorm", attn if m == "attention" else PartSpec(m, {"hidden_size": hidden}), ffn, norm, norm,
                                     f"l{i}.mixer.", f"l{i}.ffn.", f"l{i}.n1.", f"l{i}.n2.") for i, m in enumerate(mixers))
            return ModelSpec(name, vocab, hidden, 512, PartSpec("embedding", {"vocab_size": vocab, "hidden_size": hidden}),
                             layers, tuple(RunStep(i) for i in range(len(mixers))), norm,
                             PartSpec("lm_head", {"vocab_size": vocab, "hidden_size": hidden, "tied": True}),
                             embedding_prefix="emb.", final_norm_prefix="fn.", head_prefix="head.")

    return ToyConfig


def test_toy_mixer_with_two_kinds_of_state():
    """``state_need()`` gives a mapping: the previous two inputs of the sequence (a short convolution's tail, in the
    activation dtype) and the running sum of all inputs (32-bit).  Whole prompts, chunks, token by token, a batch
    of two, a reused slot and decoding from the device state must agree.  (The toy reads its metadata on the host,
    which a graph capture does not allow, so this engine launches its decode steps one by one.)"""
    from dryft_b200.cache.store import StateNeed
    from dryft_b200.config import register_architecture, unregister_architecture
    from dryft_b200.engine.api import Engine
    from dryft_b200.parts import MIXERS, TensorInfo, register_mixer
    from dryft_b200.parts.linear import linear

    class TailAndSum:
        @staticmethod
        def tensors(params, prefix):
            return {prefix + "mix.weight": TensorInfo((params["hidden_size"], params["hidden_size"]), "matrix")}

        def __init__(self, params, prefix, weights, rt):
            self.rt, self.hidden = rt, params["hidden_size"]
            self.w = weights.load(prefix + "mix.weight", "matrix")

        def kv_need(self):
            return None

        def state_need(self):
            return {"tail": StateNeed((2, self.hidden), self.rt.dtype), "sum": StateNeed((self.hidden,), torch.float32)}

        def forward(self, h, ctx, cache, state, owns_cache=True):
            # out[t] = 0.5 x[t] + 0.3 x[t-1] + 0.2 x[t-2] + mean(x[0..t]) / 4, inputs before the sequence's start are zero
            out = torch.zeros_like(h, dtype=torch.float32)
            cu, slots = ctx.cu_q.tolist(), ctx.seq_slot.tolist()
            for b, slot in enumerate(slots):
                if slot < 0:
                    continue
                x = h[cu[b]:cu[b + 1]].float()
                ext = torch.cat([state["tail"][slot].float(), x])          # [2 + n, H]: x[t-2], x[t-1] before each x[t]
                sums = state["sum"][slot][None, :] + torch.cumsum(x, dim=0)
                pos = ctx.tok_pos[cu[b]:cu[b + 1]].float()[:, None]
                out[cu[b]:cu[b + 1]] = 0.5 * ext[2:] + 0.3 * ext[1:-1] + 0.2 * ext[:-2] + sums / (pos + 1.0) / 4
                state["tail"][slot] = ext[-2:].to(state["tail"].dtype)
                state["sum"][slot] = sums[-1]
            return linear(out.to(h.dtype), self.w, self.rt)

    register_mixer("toy_tail_and_sum", TailAndSum)
    register_architecture("ToyTwoStatesForCausalLM", _toy_arch("ToyTwoStatesForCausalLM", "rmsnorm",
                                                               ["toy_tail_and_sum", "attention", "toy_tail_and_sum"], 64, 113,
                                                               heads=(2, 1, 32), inter=96))
    try:
        raw = {"architectures": ["ToyTwoStatesForCausalLM"]}
        eng = Engine.from_config(raw, seed=3, std=0.2, dtype="float32", max_batch=2, max_seq_len=128, max_tokens=256,
                                 cuda_graphs=False)
        assert isinstance(eng.cache.state(0), dict) and set(eng.cache.state(0)) == {"tail", "sum"} and eng.cache.state(1) is None
        toks = torch.randint(0, 113, (24,), generator=torch.Generator().manual_seed(0)).tolist()
        with torch.inference_mode():
            s = eng.cache.open_sequences(1)
            whole = eng.stepper.step(s, [toks], [list(range(24))]).cpu()
            eng.cache.close_sequences(s)
            s2 = eng.cache.open_sequences(1)          # the same slot again: both states start from zero
            assert s2 == s
            parts = [eng.stepper.step(s2, [toks[:7]], [list(range(7))]).cpu(), eng.stepper.step(s2, [toks[7:8]], [[0]]).cpu(),
                     eng.stepper.step(s2, [toks[8:15]], [list(range(7))]).cpu()]
            for t in toks[15:]:
                parts.append(eng.stepper.step(s2, [[t]], [[0]]).cpu())
            eng.cache.close_sequences(s2)
            s3 = eng.cache.open_sequences(2)
            both = eng.stepper.step(s3, [toks[:5], toks], [[], list(range(24))]).cpu()
            eng.cache.close_sequences(s3)
        assert torch.isfinite(whole).all() and float(whole.abs().max()) > 0
        assert H.rel_err(torch.cat(parts), whole) <= H.FP32_TOL
        assert H.rel_err(both, whole) <= H.FP32_TOL
        # generation (decode steps fed from the device state) equals feeding the same tokens by hand
        out = eng.generate_many([toks[:9]], max_new_tokens=6)[0]
        with torch.inference_mode():
            s = eng.cache.open_sequences(1)
            lg = eng.stepper.step(s, [toks[:9]], [[8]])
            for t in out:
                assert float(lg[0].max() - lg[0][t]) <= 2 * H.FP32_TOL * float(lg.abs().max())
                lg = eng.stepper.step(s, [[t]], [[0]])
            eng.cache.close_sequences(s)
    finally:
        MIXERS.unregister("toy_tail_and_sum")
        unregister_architecture("ToyTwoStatesForCausalLM")


def test_norm_of_another_arithmetic_is_never_folded_into_the_products():
    """A norm that multiplies by ``1 + w`` -- defined here in a class that is even called ``RMSNorm`` -- offers no
    ``rms_params()``: the decode step (eight rows or fewer, bfloat16, widths of 256: everything the fused products
    ask for) must run it as it is.  Decoding token by token must agree with the whole prompt (which never fuses),
    and must differ from the same weights under the stock norm."""
    from dryft_b200.config import register_architecture, unregister_architecture
    from dryft_b200.engine.api import Engine
    from dryft_b200.parts import NORMS, TensorInfo, register_norm

    class RMSNorm:   # the name is the trap
        @staticmethod
        def tensors(params, prefix):
            return {prefix + "weight": TensorInfo((params["size"],), "vector")}

        def __init__(self, params, prefix, weights, rt):
            self.eps = float(params["eps"])
            self.weight = weights.load(prefix + "weight", "vector")

        def _norm(self, x):
            xf = x.float()
            xn = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype)
            return ((1.0 + self.weight) * xn.float()).to(x.dtype)

        def forward(self, x, rows=None, n_rows=None):
            return self._norm(x if rows is None else x[rows.long()[: (n_rows if n_rows is not None else rows.numel())]])

        def add_forward(self, x, delta, rows=None, n_rows=None):
            if rows is None:
                x.copy_((x.float() + delta.float()).to(x.dtype))
                return self._norm(x)
            idx = rows.long()[: (n_rows if n_rows is not None else rows.numel())]
            return self._norm((x[idx].float() + delta[idx].float()).to(x.dtype))

    register_norm("toy_one_plus_w", RMSNorm)
    register_architecture("ToyOnePlusWForCausalLM", _toy_arch("ToyOnePlusWForCausalLM", "toy_one_plus_w", ["attention"] * 2, 256, 300))
    register_architecture("ToyStockNormForCausalLM", _toy_arch("ToyStockNormForCausalLM", "rmsnorm", ["attention"] * 2, 256, 300))
    try:
        kw = dict(seed=7, std=0.08, dtype="bfloat16", max_batch=4, max_seq_len=256, max_tokens=1024)
        toy = Engine.from_config({"architectures": ["ToyOnePlusWForCausalLM"]}, **kw)
        stock = Engine.from_config({"architectures": ["ToyStockNormForCausalLM"]}, **kw)
        toks = torch.randint(0, 300, (40,), generator=torch.Generator().manual_seed(4)).tolist()
        outs = {}
        for name, eng in (("toy", toy), ("stock", stock)):
            with torch.inference_mode():
                s = eng.cache.open_sequences(1)
                whole = eng.stepper.step(s, [toks], [list(range(20, 40))]).float().cpu()
                eng.cache.close_sequences(s)
                s = eng.cache.open_sequences(1)
                rows = [eng.stepper.step(s, [toks[:21]], [[20]])]
                for t in toks[21:]:
                    rows.append(eng.stepper.step(s, [[t]], [[0]]))
                eng.cache.close_sequences(s)
            outs[name] = (whole, torch.cat(rows).float().cpu())
        whole, stepped = outs["toy"]
        assert torch.isfinite(stepped).all()
        noise = H.rel_err(outs["stock"][1], outs["stock"][0])      # what cutting alone does in bfloat16 (stock norm)
        assert H.rel_err(stepped, whole) <= 2 * noise + 1e-3, "the toy norm was not applied as defined in the decode step"
        assert H.rel_err(stepped, outs["stock"][1]) > 20 * (2 * noise + 1e-3), "(1 + w) and w give the same logits: the test means nothing"
        # generation through the captured graph runs as well
        got = toy.generate_many([toks[:10], toks[:3]], max_new_tokens=5)
        assert [len(g) for g in got] == [5, 5]
    finally:
        NORMS.unregister("toy_one_plus_w")
        unregister_architecture("ToyOnePlusWForCausalLM")
        unregister_architecture("ToyStockNormForCausalLM")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prompts_fed_in_chunks(model_dirs, dtype):
    """``prefill_chunk_tokens``: prompts longer than the chunk go through the step function piece by piece (pieces
    that do not start on a page edge; shorter prompts finish earlier); the generated tokens are those of whole
    prompts and of the plain implementation."""
    from dryft_b200.engine.api import Engine

    name = "d"
    kw = dict(dtype=dtype, max_batch=4, max_seq_len=512, max_tokens=4 * 512)
    whole = Engine(model_dirs[name], **kw)
    chunked = Engine(model_dirs[name], prefill_chunk_tokens=50, **kw)
    prompts = H.prompts_for(name, [170, 3, 50, 51], seed=14)
    a = [s for s in whole.generate(prompts, 6)]
    b = [s for s in chunked.generate(prompts, 6)]
    plain = P.load_plain(model_dirs[name], torch.float32)
    if dtype == torch.float32:
        want = P.plain_generate(plain, prompts, 6)
        for i in range(4):
            assert [s[i] for s in a] == want[i] and [s[i] for s in b] == want[i]
    else:
        plain_b = P.load_plain(model_dirs[name], torch.bfloat16)
        for got in (a, b):
            for i, p in enumerate(prompts):
                ours = [s[i] for s in got]
                ids = list(p) + ours[:-1]
                lg = plain.logits(ids)[len(p) - 1:]
                noise = float((plain_b.logits(ids)[len(p) - 1:] - lg).abs().max())
                margin = float((lg.max(dim=-1).values - lg.gather(1, torch.tensor(ours)[:, None])[:, 0]).max())
                assert margin <= 2 * noise + 1e-3 * float(lg.abs().max())
    # the logits of a chunked prompt, against the plain model
    with torch.inference_mode():
        lg = chunked._backend._prompt_logits(chunked.cache.open_sequences(4), prompts).float().cpu()
    chunked.cache.close_sequences([0, 1, 2, 3])
    for i, p in enumerate(prompts):
        p32 = plain.logits(p)[-1:]
        if dtype == torch.float32:
            assert H.rel_err(lg[i:i + 1], p32) <= H.FP32_TOL
        else:
            pb = P.load_plain(model_dirs[name], torch.bfloat16).logits(p)[-1:]
            assert H.rel_err(lg[i:i + 1], pb) <= H.bf16_tol(pb, p32)
    with pytest.raises(ValueError):
        Engine(model_dirs[name], prefill_chunk_tokens=0, **kw)


def test_a_seed_names_one_model_wherever_it_is_drawn(tmp_path):
    """``Engine.from_config(..., draw_on="cpu")`` builds the very tensors that ``write_random_model`` stores for the
    same seed: the logits are the same bits as those of the engine loaded from the written folder, and the plain
    implementation reads the same model."""
    from dryft_b200.engine.api import Engine
    from dryft_b200.weights import write_random_model

    cfg = H.config_dict("b")
    d = write_random_model(cfg, 17, str(tmp_path / "m"), std=0.08)
    kw = dict(dtype="float32", max_batch=2, max_seq_len=128, max_tokens=256)
    from_folder = Engine(d, **kw)
    drawn = Engine.from_config(cfg, seed=17, std=0.08, draw_on="cpu", **kw)
    other = Engine.from_config(cfg, seed=17, std=0.08, draw_on="device", **kw)
    toks = H.prompts_for("b", [33], seed=2)[0]
    outs = []
    for eng in (from_folder, drawn, other):
        with torch.inference_mode():
            s = eng.cache.open_sequences(1)
            outs.append(eng.stepper.step(s, [toks], [list(range(33))]).cpu())
            eng.cache.close_sequences(s)
    assert torch.equal(outs[0], outs[1])
    assert not torch.equal(outs[0], outs[2])       # the device's generator is another one
    assert H.rel_err(outs[1], P.load_plain(d, torch.float32).logits(toks)) <= H.FP32_TOL
    with pytest.raises(ValueError):
        Engine.from_config(cfg, seed=1, draw_on="host", **kw)


def test_layers_of_other_shapes_need_no_change_to_the_library():
    """Two layer shapes that are not (norm, mixer, norm, feed-forward), in one toy architecture: a layer with a
    norm on both sides of each part (two extra norms, listed in the layer's ``extra`` and handed to a block
    arrangement registered here) and a layer without a feed-forward (the stock arrangement with ``ffn=None``).
    Whole prompts, token by token, two sequences in a batch, and a plain evaluation written out here agree."""
    from dryft_b200.config import ExtraPart, LayerSpec, ModelSpec, PartSpec, RunStep, register_architecture, unregister_architecture
    from dryft_b200.engine.api import Engine
    from dryft_b200.parts import BLOCKS, register_block
    from dryft_b200.parts.base import Residual

    class SandwichBlock:
        """x += post_m(mixer(pre_m(x)));  x += post_f(ffn(pre_f(x)))"""

        def __init__(self, norm_mixer, mixer, norm_ffn, ffn, extra):
            self.norm_mixer, self.mixer, self.norm_ffn, self.ffn = norm_mixer, mixer, norm_ffn, ffn
            self.extra = extra

        def forward(self, res, ctx, cache, state, owns_cache=True):
            x = res.x
            if res.delta is not None:
                x = (x.float() + res.delta.float()).to(x.dtype)
            a = self.extra["post_mixer"].forward(self.mixer.forward(self.norm_mixer.forward(x), ctx, cache, state, owns_cache))
            x = (x.float() + a.float()).to(x.dtype)
            f = self.extra["post_ffn"].forward(self.ffn.forward(self.norm_ffn.forward(x), ctx))
            return Residual((x.float() + f.float()).to(x.dtype))

    Hd, V, D = 48, 101, 16

    class ToyConfig:
        def __init__(self, raw):
            self.raw = dict(raw)

        def to_dict(self):
            return dict(self.raw)

        def model_spec(self):
            norm = PartSpec("rmsnorm", {"size": Hd, "eps": 1e-5})
            attn = PartSpec("attention", {"hidden_size": Hd, "num_heads": 3, "num_kv_heads": 1, "head_dim": D, "scale": 0.25,
                                          "window": None, "qk_norm": None, "position": PartSpec("rope", {"rotary_dim": D, "theta": 1e4})})
            ffn = PartSpec("swiglu", {"hidden_size": Hd, "intermediate_size": 64})
            sandwich = LayerSpec("toy_sandwich", attn, ffn, norm, norm, "l0.attn.", "l0.ffn.", "l0.pre_m.", "l0.pre_f.",
                                 extra=(ExtraPart("post_mixer", "norm", norm, "l0.post_m."), ExtraPart("post_ffn", "norm", norm, "l0.post_f.")))
            no_ffn = LayerSpec("prenorm", attn, None, norm, None, "l1.attn.", "", "l1.n.", "")
            usual = LayerSpec("prenorm", attn, ffn, norm, norm, "l2.attn.", "l2.ffn.", "l2.n1.", "l2.n2.")
            return ModelSpec("ToyShapesForCausalLM", V, Hd, 256, PartSpec("embedding", {"vocab_size": V, "hidden_size": Hd}),
                             (sandwich, no_ffn, usual), tuple(RunStep(i) for i in range(3)), norm,
                             PartSpec("lm_head", {"vocab_size": V, "hidden_size": Hd, "tied": True}),
                             embedding_prefix="emb.", final_norm_prefix="fn.", head_prefix="head.")

    register_block("toy_sandwich", SandwichBlock)
    register_architecture("ToyShapesForCausalLM", ToyConfig)
    try:
        eng = Engine.from_config({"architectures": ["ToyShapesForCausalLM"]}, seed=11, std=0.2, dtype="float32", max_batch=2,
                                 max_seq_len=128, max_tokens=256)
        n = 26
        toks = torch.randint(0, V, (n,), generator=torch.Generator().manual_seed(3)).tolist()
        with torch.inference_mode():
            s = eng.cache.open_sequences(1)
            whole = eng.stepper.step(s, [toks], [list(range(n))]).cpu()
            eng.cache.close_sequences(s)
            s = eng.cache.open_sequences(1)
            parts = [eng.stepper.step(s, [toks[:9]], [list(range(9))]).cpu()]
            for t in toks[9:]:
                parts.append(eng.stepper.step(s, [[t]], [[0]]).cpu())
            eng.cache.close_sequences(s)
            s = eng.cache.open_sequences(2)
            both = eng.stepper.step(s, [toks[:4], toks], [[3], list(range(n))]).cpu()
            eng.cache.close_sequences(s)
        assert torch.isfinite(whole).all()
        assert H.rel_err(torch.cat(parts), whole) <= H.FP32_TOL
        assert H.rel_err(both[1:], whole) <= H.FP32_TOL and H.rel_err(both[:1], whole[3:4]) <= H.FP32_TOL
        assert eng.generate_many([toks[:5]], 4)[0] == [int(t) for t in eng.generate_many([toks[:5]], 4)[0]]

        # plain evaluation from the engine's own tensors
        m = eng.model
        x = P.embed(torch.tensor(toks), m.embedding.table.float().cpu(), torch.float32)
        pos = torch.arange(n)

        def attend(at, h):
            qkv = h @ at.w_qkv.float().cpu().T
            q, k, v = qkv.split([3 * D, D, D], dim=-1)
            q, k, v = q.view(n, 3, D), k.view(n, 1, D), v.view(n, 1, D)
            cos, sin = P.rope_cos_sin(pos, D, 1e4, torch.float32)
            o = P.causal_attention(P.apply_rope(q, cos, sin), P.apply_rope(k, cos, sin), v, 0.25, None, torch.float32)
            return o @ at.w_o.float().cpu().T

        def feed(ff, h):
            gu = h @ ff.w_gate_up.float().cpu().T
            return P.silu_mul(gu[:, :64], gu[:, 64:]) @ ff.w_down.float().cpu().T

        nrm = lambda part, t: P.rmsnorm(t, part.weight.cpu(), 1e-5)
        b0, b1, b2 = m.blocks
        x = x + nrm(b0.extra["post_mixer"], attend(b0.mixer, nrm(b0.norm_mixer, x)))
        x = x + nrm(b0.extra["post_ffn"], feed(b0.ffn, nrm(b0.norm_ffn, x)))
        assert b1.ffn is None and b1.norm_ffn is None
        x = x + attend(b1.mixer, nrm(b1.norm_mixer, x))
        x = x + attend(b2.mixer, nrm(b2.norm_mixer, x))
        x = x + feed(b2.ffn, nrm(b2.norm_ffn, x))
        logits = nrm(m.final_norm, x) @ m.head.weight.float().cpu().T
        assert H.rel_err(whole, logits) <= 5 * H.FP32_TOL
    finally:
        BLOCKS.unregister("toy_sandwich")
        unregister_architecture("ToyShapesForCausalLM")
