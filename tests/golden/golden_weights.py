"""Weights and workloads of the golden cases, shared by ``make_golden.py`` and the test that reads
its output.  Self-contained: sequential draws from one seeded CPU generator, in a fixed tensor order,
rounded to bfloat16 values (held in float32) so that the 32-bit and the bfloat16 runs see the same
numbers.  The spread is wider than normal(0, 0.02): on models this small that leaves logits nearly
flat (the reference multiplies its tiny weights by 4 for the same reason, ``agent/verify.py:49-51``)."""

import torch

_A = dict(num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
          intermediate_size=128, vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
          max_position_embeddings=128)
_B = dict(num_hidden_layers=3, hidden_size=80, num_attention_heads=6, num_key_value_heads=3, head_dim=32,
          intermediate_size=224, vocab_size=384, rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
          max_position_embeddings=256)


def _prompts(lengths, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]


CASES = {
    "tiny_a": dict(config=_A, seed=0, std=0.08, prompts=_prompts([5, 9, 13], 256, 10), steps=8),
    "tiny_b": dict(config=_B, seed=1, std=0.08, prompts=_prompts([1, 7, 16, 31], 384, 11), steps=12),
}


def make_weights(c: dict, seed: int, std: float) -> dict:
    g = torch.Generator().manual_seed(seed)
    H, D, I, V = c["hidden_size"], c["head_dim"], c["intermediate_size"], c["vocab_size"]
    Hq, Hkv = c["num_attention_heads"] * D, c["num_key_value_heads"] * D

    def mat(*shape):
        return (torch.randn(*shape, generator=g) * std).to(torch.bfloat16).to(torch.float32)

    def vec(n):
        return (1.0 + torch.randn(n, generator=g) * std).to(torch.bfloat16).to(torch.float32)

    w = {"model.embed_tokens.weight": mat(V, H)}
    for i in range(c["num_hidden_layers"]):
        p = f"model.layers.{i}."
        w[p + "input_layernorm.weight"] = vec(H)
        w[p + "self_attn.q_proj.weight"] = mat(Hq, H)
        w[p + "self_attn.k_proj.weight"] = mat(Hkv, H)
        w[p + "self_attn.v_proj.weight"] = mat(Hkv, H)
        w[p + "self_attn.q_norm.weight"] = vec(D)
        w[p + "self_attn.k_norm.weight"] = vec(D)
        w[p + "self_attn.o_proj.weight"] = mat(H, Hq)
        w[p + "post_attention_layernorm.weight"] = vec(H)
        w[p + "mlp.gate_proj.weight"] = mat(I, H)
        w[p + "mlp.up_proj.weight"] = mat(I, H)
        w[p + "mlp.down_proj.weight"] = mat(H, I)
    w["model.norm.weight"] = vec(H)
    if not c["tie_word_embeddings"]:
        w["lm_head.weight"] = mat(V, H)
    return w
