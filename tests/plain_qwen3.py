"""A plain, slow implementation of the Qwen3 dense decoder, written from the formulas of
hari495/dryft's engine (each function cites ``file:line`` within that project).

Whole sequences, no cache, one function for each part.  It shares no code with
``dryft_b200``: it parses ``config.json`` and reads the safetensors file itself.  It is the
oracle of the tests; ``tests/golden/`` ties it to the reference's own model code.

Two precisions:
  * ``float32`` — every tensor and every operation in 32-bit, no rounding anywhere;
  * ``bfloat16`` — the rounding points the reference documents at
    ``engine/dryft_qwen3/model.py:4-13``: bf16 weights, activations and residual stream,
    32-bit inside norms, softmax, angles and matrix-product accumulation.  The logits are
    returned in 32-bit (the accumulator of the last product, unrounded).
"""

from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch
from safetensors import safe_open


# --------------------------------------------------------------------------- model folder
def read_model_dir(model_dir: str):
    """(config dict, {tensor name: tensor}) of a folder with config.json + model.safetensors."""
    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as f:
        cfg = json.load(f)
    tensors: Dict[str, torch.Tensor] = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt", device="cpu") as f:
        for name in f.keys():
            tensors[name] = f.get_tensor(name)
    return cfg, tensors


# --------------------------------------------------------------------------- parts
def _round(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """Round to the activation dtype; the identity in the 32-bit path."""
    return x.to(dtype)


def matmul_nt(x: torch.Tensor, w: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """``y = x @ w.T`` with 32-bit accumulation, rounded to the activation dtype
    (``F.linear``, ``engine/dryft_qwen3/model.py:153``; all weights are ``[out, in]``,
    ``OPTIMIZATION_GUIDE.md:117``)."""
    return _round(x.to(torch.float32) @ w.to(torch.float32).T, dtype)


def embed(ids: torch.Tensor, table: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """``x = embed[ids]`` (``engine/dryft_qwen3/model.py:132``)."""
    return _round(table[ids], dtype)


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """``w * cast(x32 * rsqrt(mean(x32^2) + eps))``: the weight multiplies AFTER the cast back
    (``engine/dryft_qwen3/model.py:28-32``)."""
    xf = x.to(torch.float32)
    var = xf.pow(2).mean(-1, keepdim=True)
    xn = (xf * torch.rsqrt(var + eps)).to(x.dtype)
    return (w.to(torch.float32) * xn.to(torch.float32)).to(x.dtype)


def rope_cos_sin(positions: torch.Tensor, head_dim: int, theta: float, dtype: torch.dtype):
    """cos/sin ``[T, head_dim]``: ``inv_freq = 1/theta^(2j/D)``, angles in 32-bit, the two halves
    equal (``cat(freqs, freqs)``), then cast to the activation dtype
    (``engine/dryft_qwen3/model.py:49-57``)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.int64).to(torch.float32) / head_dim))
    freqs = positions.to(torch.float32)[:, None] * inv_freq[None, :]
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """``cat(-x[D/2:], x[:D/2])`` (``engine/dryft_qwen3/model.py:35-37``)."""
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """``x*cos + rotate_half(x)*sin`` in the activation dtype: in bf16 every product and the sum
    round (``engine/dryft_qwen3/model.py:40-41``; ``kernels/rope_qknorm.py:15-20``).
    x ``[T, heads, D]``, cos/sin ``[T, D]``."""
    c = cos[:, None, :]
    s = sin[:, None, :]
    return (x * c) + (rotate_half(x) * s)


def causal_attention(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: Optional[int], dtype: torch.dtype
) -> torch.Tensor:
    """Grouped-query causal attention of one sequence.  q ``[T, nH, D]``, k/v ``[T, nKV, D]``;
    q head ``h`` uses kv head ``h // G``; key ``j`` is visible to query ``i`` iff ``j <= i`` (and
    ``i - j < window`` when a window is set); scores and softmax in 32-bit
    (``engine/dryft_qwen3/model.py:172-178,235,254-258``; ``kernels/attn_decode.py:180-196``)."""
    T, nH, D = q.shape
    nKV = k.shape[1]
    G = nH // nKV
    qf = q.to(torch.float32).view(T, nKV, G, D)
    kf = k.to(torch.float32)
    vf = v.to(torch.float32)
    scores = torch.einsum("ihgd,jhd->hgij", qf, kf) * scale
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    visible = j <= i
    if window is not None:
        visible = visible & (i - j < window)
    scores = scores.masked_fill(~visible, float("-inf"))
    p = torch.softmax(scores, dim=-1)
    o = torch.einsum("hgij,jhd->ihgd", p, vf).reshape(T, nH * D)
    return _round(o, dtype)


def silu_mul(g: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    """``cast(silu32(g)) * u`` with ``silu(t) = t/(1+exp(-t))``: the silu is rounded to the
    activation dtype before the product (``engine/dryft_qwen3/model.py:44-46``;
    ``kernels/silu_mul.py:4-5,29-32``)."""
    gf = g.to(torch.float32)
    s = (gf / (1.0 + torch.exp(-gf))).to(g.dtype)
    return (s.to(torch.float32) * u.to(torch.float32)).to(g.dtype)


def swiglu(h: torch.Tensor, w_gate, w_up, w_down, dtype: torch.dtype) -> torch.Tensor:
    """``down(silu(gate(h)) * up(h))`` (``engine/dryft_qwen3/model.py:180``)."""
    g = matmul_nt(h, w_gate, dtype)
    u = matmul_nt(h, w_up, dtype)
    return matmul_nt(silu_mul(g, u), w_down, dtype)


def residual_add(x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """``x + y``: summed in 32-bit, rounded once to the stream's dtype
    (``kernels/rmsnorm.py:34``)."""
    return (x.to(torch.float32) + y.to(torch.float32)).to(x.dtype)


# --------------------------------------------------------------------------- whole model
class PlainQwen3:
    """Whole-sequence forward pass; no state between calls."""

    def __init__(self, cfg: dict, tensors: Dict[str, torch.Tensor], dtype: torch.dtype):
        assert dtype in (torch.float32, torch.bfloat16)
        self.dtype = dtype
        self.L = int(cfg["num_hidden_layers"])
        self.H = int(cfg["hidden_size"])
        self.nH = int(cfg["num_attention_heads"])
        self.nKV = int(cfg["num_key_value_heads"])
        self.D = int(cfg.get("head_dim") or self.H // self.nH)  # config.py:142
        self.I = int(cfg["intermediate_size"])
        self.V = int(cfg["vocab_size"])
        self.eps = float(cfg["rms_norm_eps"])
        self.theta = float(cfg["rope_theta"])
        self.tied = bool(cfg.get("tie_word_embeddings", False))  # config.py:153
        self.scale = 1.0 / math.sqrt(self.D)  # model.py:65
        self.windows: List[Optional[int]] = [None] * self.L
        if cfg.get("use_sliding_window", False):
            types = cfg.get("layer_types")
            if types is None:
                first = cfg.get("max_window_layers", self.L)
                types = ["sliding_attention" if i >= first else "full_attention" for i in range(self.L)]
            self.windows = [int(cfg["sliding_window"]) if t == "sliding_attention" else None for t in types]
        # 32-bit path: every tensor upcast (exact); bf16 path: tensors as stored
        self.t = {k: (v.to(torch.float32) if dtype == torch.float32 else v) for k, v in tensors.items()}

    def w(self, name: str) -> torch.Tensor:
        return self.t[name]

    def hidden_states(self, ids: Sequence[int]) -> torch.Tensor:
        """Residual stream after the last layer, ``[T, H]`` (``model.py:132-184``)."""
        dt = self.dtype
        idt = torch.tensor(list(ids), dtype=torch.int64)
        T = idt.numel()
        x = embed(idt, self.w("model.embed_tokens.weight"), dt)
        cos, sin = rope_cos_sin(torch.arange(T), self.D, self.theta, dt)
        for i in range(self.L):
            p = f"model.layers.{i}."
            h = rmsnorm(x, self.w(p + "input_layernorm.weight"), self.eps)  # model.py:151
            q = matmul_nt(h, self.w(p + "self_attn.q_proj.weight"), dt).view(T, self.nH, self.D)
            k = matmul_nt(h, self.w(p + "self_attn.k_proj.weight"), dt).view(T, self.nKV, self.D)
            v = matmul_nt(h, self.w(p + "self_attn.v_proj.weight"), dt).view(T, self.nKV, self.D)
            q = rmsnorm(q, self.w(p + "self_attn.q_norm.weight"), self.eps)  # model.py:165
            k = rmsnorm(k, self.w(p + "self_attn.k_norm.weight"), self.eps)  # model.py:166
            q = apply_rope(q, cos, sin)  # model.py:168-169
            k = apply_rope(k, cos, sin)
            o = causal_attention(q, k, v, self.scale, self.windows[i], dt)
            x = residual_add(x, matmul_nt(o, self.w(p + "self_attn.o_proj.weight"), dt))  # model.py:179
            h = rmsnorm(x, self.w(p + "post_attention_layernorm.weight"), self.eps)
            m = swiglu(
                h,
                self.w(p + "mlp.gate_proj.weight"),
                self.w(p + "mlp.up_proj.weight"),
                self.w(p + "mlp.down_proj.weight"),
                dt,
            )
            x = residual_add(x, m)  # model.py:181-184
        return x

    def logits(self, ids: Sequence[int]) -> torch.Tensor:
        """32-bit logits at every position, ``[T, V]``: final norm, then the output head, which is
        the embedding table when tied (``model.py:185-186``; ``weights.py:47-49``)."""
        x = self.hidden_states(ids)
        h = rmsnorm(x, self.w("model.norm.weight"), self.eps)
        head = self.w("model.embed_tokens.weight") if self.tied else self.w("lm_head.weight")
        return h.to(torch.float32) @ head.to(torch.float32).T


def load_plain(model_dir: str, dtype: torch.dtype) -> PlainQwen3:
    cfg, tensors = read_model_dir(model_dir)
    return PlainQwen3(cfg, tensors, dtype)


# --------------------------------------------------------------------------- token choice
_MASK64 = (1 << 64) - 1


def uniform_draw(seed: int, sequence: int, step: int) -> float:
    """The library's counter-based uniform in [0, 1): a 64-bit mix of (seed, sequence index,
    step), top 24 bits.  The reference samples nothing (``model.py:187`` is an argmax); this
    restates the library's own definition independently, in Python integers."""
    z = (seed * 0x9E3779B97F4A7C15 + sequence * 0xBF58476D1CE4E5B9 + step * 0x94D049BB133111EB + 0x2545F4914F6CDD1D) & _MASK64
    z ^= z >> 30
    z = (z * 0xBF58476D1CE4E5B9) & _MASK64
    z ^= z >> 27
    z = (z * 0x94D049BB133111EB) & _MASK64
    z ^= z >> 31
    return (z >> 40) / float(1 << 24)


def choose_token(logits: torch.Tensor, temperature: float, top_k: int, u: float) -> int:
    """Greedy: the first index of the maximum (``model.py:187``; ``AGENTS.md:174-175``).
    Otherwise keep the ``top_k`` largest logits (ties to the lower index; 0 keeps all), divide by
    the temperature, softmax in 32-bit, and take the first kept index, in index order, whose
    running sum of probabilities exceeds ``u``."""
    lg = logits.to(torch.float32)
    V = lg.numel()
    if temperature <= 0.0:
        return int(torch.argmax(lg).item())
    keep = torch.ones(V, dtype=torch.bool)
    if 0 < top_k < V:
        # stable descending sort: equal logits keep index order, so ties go to the lower index
        order = torch.sort(lg, descending=True, stable=True).indices
        keep = torch.zeros(V, dtype=torch.bool)
        keep[order[:top_k]] = True
    z = lg / torch.tensor(temperature, dtype=torch.float32)
    z = torch.where(keep, z, torch.tensor(float("-inf")))
    e = torch.exp(z - z.max())
    total = e.sum()
    cdf = torch.cumsum(e, dim=0)
    hit = torch.nonzero((cdf > u * total) & keep)
    if hit.numel() == 0:
        return int(torch.nonzero(keep)[-1].item())
    return int(hit[0].item())


def plain_generate(
    model: PlainQwen3,
    prompts: Sequence[Sequence[int]],
    max_new_tokens: int,
    temperature: float = 0.0,
    top_k: int = 0,
    seed: int = 0,
    stop_token_ids: Sequence[int] = (),
) -> List[List[int]]:
    """Each sequence alone, re-running the whole sequence for every new token.  Sequence ``b``
    draws with ``uniform_draw(seed, b, step)``; a stop token is kept and ends the sequence."""
    out: List[List[int]] = []
    for b, prompt in enumerate(prompts):
        ids = list(prompt)
        new: List[int] = []
        for step in range(max_new_tokens):
            lg = model.logits(ids)[-1]
            tok = choose_token(lg, temperature, top_k, uniform_draw(seed, b, step))
            new.append(tok)
            ids.append(tok)
            if tok in stop_token_ids:
                break
        out.append(new)
    return out
