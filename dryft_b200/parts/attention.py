"""Grouped-query attention over the paged cache, the mixer of every Qwen3 layer.

Per step (``engine/dryft_qwen3/model.py:153-179,237-258``):
  ``qkv = h @ W_qkv.T`` (rows q; k; v fused, ``weights.py:93-96``) -> per-head RMSNorm of q and k
  (before RoPE, ``model.py:165-166``) -> rotate-half RoPE at each token's own position -> K and V
  written into the cache at that position (``model.py:170-171,249-250``) -> attention of every query
  token over keys ``0..its position`` of its own sequence (``model.py:235``), q head ``h`` reading kv
  head ``h // G`` -> ``@ W_o.T``.

The three middle stages are one kernel (``csrc/rope_kv.cu``); attention is ``csrc/attn_prefill.cu``
(bfloat16 prompts, tensor cores) or ``csrc/attn_rows.cu`` (decode, and everything in 32-bit).
Every size and constant is a parameter: head counts, head size, scale, eps, window, rotary part.
"""

from __future__ import annotations

import math
from typing import Dict, Mapping, Optional

import torch

from ..cache.store import CacheEntry, KVNeed, StateNeed
from ..config.spec import PartSpec
from ..ops import kernels as K
from .base import NORMS, POSITIONS, Runtime, StepContext, TensorInfo, fused_rms, register_mixer
from .linear import fusable_rows, linear, weighted_for

PREFILL_TILE = 64      # query rows per block of the mma.sync prefill kernel
PREFILL_TILE_TC = 128  # query rows per block of the tcgen05 prefill kernel


@register_mixer("attention")
class Attention:
    @staticmethod
    def tensors(params: Mapping, prefix: str) -> Dict[str, TensorInfo]:
        h, nh, nkv, d = params["hidden_size"], params["num_heads"], params["num_kv_heads"], params["head_dim"]
        t = {
            prefix + "q_proj.weight": TensorInfo((nh * d, h), "matrix"),
            prefix + "k_proj.weight": TensorInfo((nkv * d, h), "matrix"),
            prefix + "v_proj.weight": TensorInfo((nkv * d, h), "matrix"),
            prefix + "o_proj.weight": TensorInfo((h, nh * d), "matrix"),
        }
        qk = params.get("qk_norm")
        if qk is not None:
            t.update(NORMS.get(qk.kind).tensors(qk.params, prefix + "q_norm."))
            t.update(NORMS.get(qk.kind).tensors(qk.params, prefix + "k_norm."))
        return t

    def __init__(self, params: Mapping, prefix: str, weights, rt: Runtime):
        self.rt = rt
        self.hidden = int(params["hidden_size"])
        self.n_heads = int(params["num_heads"])
        self.n_kv = int(params["num_kv_heads"])
        self.head_dim = int(params["head_dim"])
        self.scale = float(params["scale"])
        self.window: Optional[int] = params.get("window")
        if self.n_heads % self.n_kv:
            raise ValueError(f"attention: {self.n_heads} heads are not a multiple of {self.n_kv} kv heads")
        self.group = self.n_heads // self.n_kv
        self.q_dim = self.n_heads * self.head_dim
        self.kv_dim = self.n_kv * self.head_dim
        names = [prefix + f"{p}_proj.weight" for p in ("q", "k", "v")]
        self.w_qkv = weights.load_fused(names, [self.q_dim, self.kv_dim, self.kv_dim], self.hidden)
        self.w_o = weights.load(prefix + "o_proj.weight", "matrix")
        qk: Optional[PartSpec] = params.get("qk_norm")
        self.qk_eps = 0.0
        self.q_norm_w = self.k_norm_w = None
        if qk is not None:
            if qk.kind != "rmsnorm" or int(qk["size"]) != self.head_dim:
                raise ValueError("attention: the per-head q/k norm must be an rmsnorm over head_dim")
            self.qk_eps = float(qk["eps"])
            self.q_norm_w = weights.load(prefix + "q_norm.weight", "vector")
            self.k_norm_w = weights.load(prefix + "k_norm.weight", "vector")
        pos: PartSpec = params.get("position") or PartSpec("none")
        self.position = POSITIONS.get(pos.kind)(pos.params, self.head_dim, rt)
        # build (or find) the kernels this head shape needs now, not at the first step
        K.attention_rows_lib(self.head_dim, self.group, rt.page_size)
        self.use_prefill_kernel = rt.is_bf16
        self.use_decode_kernel = rt.is_bf16 and rt.fuse_decode and K.attention_decode_supported(self.head_dim, self.group)
        # prompts: tcgen05 / TMEM / TMA where the head size allows, else mma.sync
        self.use_prefill_tc = rt.is_bf16 and rt.tcgen05 and K.attention_prefill_tc_supported(self.head_dim, self.group, rt.page_size)
        self.prefill_tile = PREFILL_TILE_TC if self.use_prefill_tc else PREFILL_TILE
        if self.use_prefill_tc:
            K.attention_prefill_tc_lib(self.head_dim, self.group, rt.page_size)
        if self.use_prefill_kernel:
            K.attention_prefill_lib(self.head_dim, self.group, rt.page_size)
        if self.use_decode_kernel:
            K.attention_decode_lib(self.head_dim, self.group, rt.page_size)

    def kv_need(self) -> Optional[KVNeed]:
        return KVNeed(self.n_kv, self.head_dim, self.window)

    def state_need(self) -> Optional[StateNeed]:
        return None

    def _n_splits(self, n_rows: int) -> int:
        """Split the keys of each row over enough blocks to fill the device (the reference aims at
        two programs per SM, ``kernels/attn_decode.py:143-149``)."""
        want = math.ceil(2 * self.rt.sm_count / max(1, n_rows * self.n_kv))
        return max(1, min(32, want))

    CLUSTER_SPLITS = 8   # up to this many splits run as one thread-block cluster (combined on chip)

    def _decode_splits(self, max_kv: int, n_rows: int) -> int:
        """Splits of the one-launch decode attention.  Up to eight splits of a (row, kv head) run as one
        thread-block cluster and are combined through distributed shared memory, which costs about a
        microsecond, so a block may take as little as three pages (192 keys: one or two 16-key slices per
        warp) -- as long as the grid stays within one block per SM: more blocks than that take the slots in
        which the next launch's blocks start early, which costs more than the shorter walk saves.
        Sequences too long for that split further and meet in memory (a block then takes up to 1,024 keys)."""
        pages = (max(1, max_kv) + self.rt.page_size - 1) // self.rt.page_size
        room = max(1, self.rt.sm_count // max(1, n_rows * self.n_kv))
        by_cluster = min((pages + 2) // 3, room, self.CLUSTER_SPLITS)
        if by_cluster > 4 and n_rows * self.n_kv > 8:
            # a cluster of 5..8 blocks (one block a SM) needs that many free SMs in one GPC: with more than
            # eight such clusters some wait for a whole GPC's worth of SMs (batch 2 at 2,063 keys: 20.8 us a
            # layer with 16 clusters of 8 against 12.9 us with 16 clusters of 4)
            by_cluster = 4
        by_memory = min(32, (max(1, max_kv) + 1023) // 1024)
        if by_memory > self.CLUSTER_SPLITS:
            # also within one block per SM where the batch allows it (batch 1 at 32,768 keys: 18 splits, not 32:
            # measured inside the step 1.1 ms of 4.3 ms faster, although 32 splits are faster when timed alone)
            by_memory = min(by_memory, max(room, self.CLUSTER_SPLITS))
        return max(1, by_cluster) if by_memory <= self.CLUSTER_SPLITS else by_memory

    def can_fuse(self, n_rows: int, norm) -> bool:
        """Few rows, bfloat16 everywhere, widths the weight-streaming product takes."""
        rt = self.rt
        return (rt.fuse_decode and rt.is_bf16 and fusable_rows(n_rows, self.hidden, rt, normed=True) and fusable_rows(n_rows, self.q_dim, rt)
                and fused_rms(norm) is not None and self.w_qkv.dtype == torch.bfloat16 and self.w_o.dtype == torch.bfloat16)

    weighted_ahead = True   # forward_normed takes ``xw`` / ``next_norm`` and returns the weighted stream too

    def forward_normed(self, x, ss, ss_parts, norm, ctx, cache, state, owns_cache: bool = True, xw=None, next_norm=None):
        """``x += o_proj(attention(qkv_proj(norm(x))))`` in place: the norm inside the first product,
        the add inside the last, which also leaves the new sums of squares of ``x``.  ``xw``: ``x`` weighted
        by ``norm``'s weight already (the first product then has no prologue).  ``next_norm``: the norm that
        reads ``x`` next; the last product leaves ``x`` weighted for it where the sizes allow.
        Returns ``(ss, ss_parts, xw or None)``."""
        n = x.shape[0]
        w = self.w_qkv if owns_cache else self.w_qkv[: self.q_dim]
        qkv = torch.empty((n, w.shape[0]), dtype=x.dtype, device=x.device)
        norm_w, eps = fused_rms(norm)
        small = self.rt.small_m_max
        if xw is not None and K.weighted_ahead_supported(self.hidden):
            K.fused_product(x, w, qkv, small_m_max=small, xw_in=xw, norm_w=norm_w, ss_in=ss, ss_parts=ss_parts, eps=eps, pdl=self.rt.pdl)
        else:
            K.fused_product(x, w, qkv, small_m_max=small, norm_w=norm_w, ss_in=ss, ss_parts=ss_parts, eps=eps, pdl=self.rt.pdl)
        o = self._attend(qkv, ctx, cache, owns_cache)
        parts = K.fused_ss_parts(n, self.hidden, self.q_dim, small)
        ss_out = torch.empty(parts * K.SS_STRIDE, dtype=torch.float32, device=x.device)
        xw_out = None
        if weighted_for(next_norm, self.hidden, self.q_dim, self.rt, n):
            xw_out = torch.empty_like(x)
            K.fused_product(o, self.w_o, x, small_m_max=small, mode="residual", ss_out=ss_out, pdl=self.rt.pdl,
                            next_w=fused_rms(next_norm)[0], xw_out=xw_out)
        else:
            K.fused_product(o, self.w_o, x, small_m_max=small, mode="residual", ss_out=ss_out, pdl=self.rt.pdl)
        return ss_out, parts, xw_out

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: CacheEntry, state, owns_cache: bool = True) -> torch.Tensor:
        if owns_cache:
            qkv = linear(h, self.w_qkv, self.rt)
        else:  # a run step that reads another step's cache projects queries only
            qkv = linear(h, self.w_qkv[: self.q_dim], self.rt)
        return linear(self._attend(qkv, ctx, cache, owns_cache), self.w_o, self.rt)

    def _attend(self, qkv: torch.Tensor, ctx: StepContext, cache: CacheEntry, owns_cache: bool) -> torch.Tensor:
        """q/k norm + RoPE + cache write, then attention over the cache: ``[tokens, q_dim]``."""
        n = qkv.shape[0]
        dev = qkv.device
        h = qkv
        if ctx.decode and self.use_decode_kernel:
            # one launch: q/k norm + RoPE + cache write + split attention + combine
            o = torch.empty((n, self.q_dim), dtype=h.dtype, device=dev)
            s = self._decode_splits(ctx.max_kv, n)
            part_o = part_ml = None
            if s > self.CLUSTER_SPLITS:
                part_o = torch.empty((n, self.n_heads, s, self.head_dim), dtype=torch.float32, device=dev)
                part_ml = torch.empty((n, self.n_heads, s, 2), dtype=torch.float32, device=dev)
            K.attn_decode(qkv, self.q_norm_w, self.k_norm_w, self.position.inv_freq, ctx.tok_slot, ctx.tok_pos, cache.k, cache.v,
                          cache.page_table, o, self.n_heads, self.n_kv, self.head_dim, self.position.rotary_dim, self.qk_eps,
                          self.scale, self.window, s, part_o, part_ml, write_kv=owns_cache, pdl=self.rt.pdl)
            return o
        q = torch.empty((n, self.n_heads, self.head_dim), dtype=h.dtype, device=dev)
        table_of = getattr(self.position, "table", None)   # a step of many tokens shares its cos / sin between layers
        K.qk_norm_rope_store(qkv, self.q_norm_w, self.k_norm_w, self.position.inv_freq, ctx.tok_slot, ctx.tok_pos, q,
                             cache.k, cache.v, cache.page_table, self.n_heads, self.n_kv, self.head_dim,
                             self.position.rotary_dim, self.qk_eps, write_kv=owns_cache,
                             cs_table=table_of(ctx) if table_of is not None else None,
                             zero_tail=owns_cache and not ctx.decode and (self.use_prefill_tc or self.use_prefill_kernel))
        o = torch.empty((n, self.q_dim), dtype=h.dtype, device=dev)
        if self.use_prefill_tc and not ctx.decode and ctx.n_tiles > 0 and ctx.tile_size <= PREFILL_TILE_TC:
            K.attn_prefill_tc(q, cache.k, cache.v, cache.page_table, ctx.tile_tok0, ctx.tile_rows, ctx.tok_slot, ctx.tok_pos,
                              o, ctx.n_tiles, self.scale, self.window)
        elif self.use_prefill_kernel and not ctx.decode and ctx.n_tiles > 0 and ctx.tile_size <= PREFILL_TILE:
            K.attn_prefill(q, cache.k, cache.v, cache.page_table, ctx.tile_tok0, ctx.tile_rows, ctx.tok_slot, ctx.tok_pos,
                           o, ctx.n_tiles, self.scale, self.window)
        else:
            s = self._n_splits(n)
            part_o = part_ml = None
            if s > 1:
                part_o = torch.empty((n, self.n_heads, s, self.head_dim), dtype=torch.float32, device=dev)
                part_ml = torch.empty((n, self.n_heads, s, 2), dtype=torch.float32, device=dev)
            K.attn_rows(q, cache.k, cache.v, cache.page_table, ctx.tok_slot, ctx.tok_pos, o, self.scale, self.window,
                        s, part_o, part_ml)
        return o
