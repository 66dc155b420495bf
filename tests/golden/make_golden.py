"""Makes ``tests/golden/*.safetensors``: logits of hari495/dryft's OWN model code on the CPU, for
the plain implementation (``tests/plain_qwen3.py``) to be compared with once.

    python tests/golden/make_golden.py [/path/to/hari495-dryft]      (default: $DRYFT_REFERENCE)

How the reference is driven (nothing in its tree is changed):
  * ``dryft_qwen3.config.EXPECTED_CONFIG = None`` lifts the pin to one checkpoint
    (``engine/dryft_qwen3/config.py:55-70,121-135``), as its own ``agent/verify.py:61`` does.
  * ``Model.prefill`` / ``Model.decode_step`` (``engine/dryft_qwen3/model.py:123,191``) are called
    directly with hand-built ``Weights``; a subclass returns a separate ``lm_head`` for the untied
    configuration (``weights.py:47-49`` only knows the tied case).
  * The reference never returns logits (``model.py:187,262`` take the argmax); they are captured by
    wrapping ``F.linear`` inside ``dryft_qwen3.model`` and keeping the call whose weight is the head.
  * 32-bit: float32 weights, float32 cos/sin tables built with the expression of ``model.py:49-57``
    (without its final cast), float32 caches.  bfloat16: everything as the reference has it.
Each case: ragged prompts prefilled one by one, then greedy decode steps of the whole batch; the
file holds the prompts, the greedy tokens and the logits of every step.
The weights are drawn by ``golden_weights.make_weights`` (sequential draws from one seeded CPU
generator), which the test calls again, so no weights are stored.
"""

import os
import sys

import torch
from safetensors.torch import save_file

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from golden_weights import CASES, make_weights  # noqa: E402


def run_case(ref_root: str, case: dict, dtype: torch.dtype):
    sys.path.insert(0, os.path.join(ref_root, "engine"))
    from dryft_qwen3 import config as C
    from dryft_qwen3 import model as M
    from dryft_qwen3.cache import DecodeState
    from dryft_qwen3.weights import LayerWeights, Weights

    C.EXPECTED_CONFIG = None
    c = case["config"]
    cfg = C.ModelConfig(num_layers=c["num_hidden_layers"], hidden=c["hidden_size"], num_heads=c["num_attention_heads"],
                        num_kv_heads=c["num_key_value_heads"], head_dim=c["head_dim"], intermediate=c["intermediate_size"],
                        vocab=c["vocab_size"], eps=c["rms_norm_eps"], rope_theta=c["rope_theta"],
                        tie_embeddings=c["tie_word_embeddings"], max_position=c["max_position_embeddings"])
    w = {k: v.to(dtype) for k, v in make_weights(c, case["seed"], case["std"]).items()}
    layers = []
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        layers.append(LayerWeights(
            w_in=w[p + "input_layernorm.weight"],
            w_qkv=torch.cat([w[p + "self_attn.q_proj.weight"], w[p + "self_attn.k_proj.weight"], w[p + "self_attn.v_proj.weight"]]),
            w_qn=w[p + "self_attn.q_norm.weight"], w_kn=w[p + "self_attn.k_norm.weight"],
            w_o=w[p + "self_attn.o_proj.weight"], w_post=w[p + "post_attention_layernorm.weight"],
            w_gu=torch.cat([w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"]]),
            w_down=w[p + "mlp.down_proj.weight"]))

    class HeadWeights(Weights):
        head = None

        @property
        def lm_head(self):
            return self.head

    weights = HeadWeights(embed=w["model.embed_tokens.weight"], layers=layers, norm=w["model.norm.weight"])
    weights.head = w["model.embed_tokens.weight"] if cfg.tie_embeddings else w["lm_head.weight"]

    L = 64
    dev = torch.device("cpu")
    mdl = M.Model(cfg, weights, dev, rope_len=L)
    if dtype == torch.float32:
        d = cfg.head_dim
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, d, 2, dtype=torch.int64).to(torch.float32) / d))
        fr = torch.arange(L, dtype=torch.float32)[:, None] * inv[None, :]
        emb = torch.cat((fr, fr), dim=-1)
        rope = (emb.cos(), emb.sin())
    else:
        rope = (mdl.cos, mdl.sin)
    B = len(case["prompts"])
    st = DecodeState(cfg, B, L, dev, pinned=False, rope=rope)
    st.k_cache = st.k_cache.to(dtype)
    st.v_cache = st.v_cache.to(dtype)

    captured = []
    orig = M.F.linear

    def spy(x, wt, *a, **k):
        y = orig(x, wt, *a, **k)
        if wt is weights.head and wt.shape[0] == cfg.vocab and x.shape[-1] == cfg.hidden and not captured_off[0]:
            captured.append(y.detach().clone())
        return y

    captured_off = [False]
    M.F.linear = spy
    try:
        out = {}
        toks = []
        pre = []
        for r, p in enumerate(case["prompts"]):
            n0 = len(captured)
            nxt = mdl.prefill(st, torch.tensor([r]), torch.tensor([p], dtype=torch.int64))
            pre.append(captured[-1].reshape(-1).float())
            assert len(captured) == n0 + 1
            st.ids[r] = nxt[0]
            st.seq_lens[r] = len(p)
        out["prefill_logits"] = torch.stack(pre)
        toks.append(st.ids[:B].clone())
        dec = []
        for _ in range(case["steps"] - 1):
            mdl.decode_step(st, B, L)
            dec.append(captured[-1].float())
            toks.append(st.next_ids[:B].clone())
        out["decode_logits"] = torch.stack(dec)
        out["tokens"] = torch.stack(toks).to(torch.int32)
    finally:
        M.F.linear = orig
    return out


def main() -> int:
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("DRYFT_REFERENCE", "")
    if not ref:
        raise SystemExit("give the path of a checkout of hari495/dryft (argument or $DRYFT_REFERENCE)")
    if not os.path.isdir(os.path.join(ref, "engine", "dryft_qwen3")):
        print(f"reference not found at {ref}", file=sys.stderr)
        return 1
    for name, case in CASES.items():
        for dtype, tag in ((torch.float32, "f32"), (torch.bfloat16, "bf16")):
            out = run_case(ref, case, dtype)
            path = os.path.join(HERE, f"{name}_{tag}.safetensors")
            save_file({k: v.contiguous() for k, v in out.items()}, path)
            print(path, {k: tuple(v.shape) for k, v in out.items()})
    return 0


if __name__ == "__main__":
    sys.exit(main())
