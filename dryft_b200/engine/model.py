"""A decoder put together from a ``ModelSpec``: embedding, the layers' blocks in run order, final
norm and output head.  It is the same class for every architecture; what differs is the spec.

One forward pass serves prefill and decode: it runs exactly the tokens of the step, reads and writes
the cache through each run step's ``CacheEntry``, and returns 32-bit logits at the wanted rows only
(the reference computes the last position only and returns its argmax,
``engine/dryft_qwen3/model.py:185-187,261-262``).
"""

from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from ..cache.store import KVNeed, SequenceCache, StateNeed
from ..config.spec import ModelSpec
from ..parts.base import BLOCKS, EMBEDDINGS, FAMILIES, FFNS, HEADS, MIXERS, NORMS, Residual, Runtime, StepContext


class DecoderModel:
    def __init__(self, spec: ModelSpec, weights, rt: Runtime):
        spec.validate()
        self.spec = spec
        self.rt = rt
        self.vocab_size = spec.vocab_size
        self.hidden_size = spec.hidden_size
        self.embedding = EMBEDDINGS.get(spec.embedding.kind)(spec.embedding.params, spec.embedding_prefix, weights, rt)
        self.blocks = []
        for layer in spec.layers:
            norm_mixer = NORMS.get(layer.norm_mixer.kind)(layer.norm_mixer.params, layer.norm_mixer_prefix, weights, rt)
            mixer = MIXERS.get(layer.mixer.kind)(layer.mixer.params, layer.mixer_prefix, weights, rt)
            norm_ffn = ffn = None
            if layer.ffn is not None:
                norm_ffn = NORMS.get(layer.norm_ffn.kind)(layer.norm_ffn.params, layer.norm_ffn_prefix, weights, rt)
                ffn = FFNS.get(layer.ffn.kind)(layer.ffn.params, layer.ffn_prefix, weights, rt)
            extra = {e.name: FAMILIES[e.family].get(e.spec.kind)(e.spec.params, e.prefix, weights, rt) for e in layer.extra}
            make = BLOCKS.get(layer.block)
            self.blocks.append(make(norm_mixer, mixer, norm_ffn, ffn, extra=extra) if extra else make(norm_mixer, mixer, norm_ffn, ffn))
        self.final_norm = NORMS.get(spec.final_norm.kind)(spec.final_norm.params, spec.final_norm_prefix, weights, rt)
        self.head = HEADS.get(spec.head.kind)(spec.head.params, spec.head_prefix, weights, rt, embedding=self.embedding)

    # what each run step asks of the cache
    def cache_needs(self) -> Tuple[List[Tuple[Optional[KVNeed], Optional[StateNeed]]], List[Optional[int]]]:
        needs, borrow = [], []
        for st in self.spec.schedule:
            mixer = self.blocks[st.layer].mixer
            needs.append((mixer.kv_need(), mixer.state_need()))
            borrow.append(st.cache_from)
        return needs, borrow

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        def visit(obj):
            nonlocal total
            for v in vars(obj).values():
                if isinstance(v, torch.Tensor) and v.is_floating_point() and v.dim() >= 1:
                    key = v.data_ptr()
                    if key not in seen:
                        seen.add(key)
                        total += v.numel() * v.element_size()
        visit(self.embedding); visit(self.final_norm); visit(self.head)
        for b in self.blocks:
            for part in (b.norm_mixer, b.mixer, b.norm_ffn, b.ffn, *getattr(b, "extra", {}).values()):
                if part is not None:
                    visit(part)
        return total

    def forward(self, ctx: StepContext, cache: SequenceCache, want_rows: Optional[torch.Tensor], n_want: int,
                all_rows: bool = False) -> Optional[torch.Tensor]:
        """Run the step's tokens through every run step; logits ``[n_want, vocab]`` float32 at the
        packed rows ``want_rows`` (None if nothing is wanted).  ``all_rows`` says that ``want_rows`` is simply
        every row in order (a decode step), which lets the head take the fused path."""
        res = Residual(self.embedding.forward(ctx.tokens, ctx.n_tokens))
        sched = self.spec.schedule
        for i, st in enumerate(sched):
            block = self.blocks[st.layer]
            if getattr(block, "takes_next_norm", False):
                # the norm that reads the stream next: the following run step's first norm, or the final norm
                nxt = getattr(self.blocks[sched[i + 1].layer], "norm_mixer", None) if i + 1 < len(sched) else self.final_norm
                res = block.forward(res, ctx, cache.entry(i), cache.state(i), owns_cache=st.cache_from is None, next_norm=nxt)
            else:
                res = block.forward(res, ctx, cache.entry(i), cache.state(i), owns_cache=st.cache_from is None)
        if n_want == 0:
            return None
        if (all_rows and res.delta is None and res.ss is not None and hasattr(self.head, "forward_normed")
                and self.head.can_fuse(res.x.shape[0], self.final_norm)):
            xw = res.xw if res.xw_norm is self.final_norm else None
            return self.head.forward_normed(res.x, res.ss, res.ss_parts, self.final_norm, **({"xw": xw} if xw is not None else {}))
        if res.delta is None:
            h = self.final_norm.forward(res.x, rows=want_rows, n_rows=n_want)
        else:
            h = self.final_norm.add_forward(res.x, res.delta, rows=want_rows, n_rows=n_want)
        return self.head.forward(h)
