"""What every part of a layer has in common: the registries that map a ``PartSpec.kind`` to a class,
the description of the tensors a part reads from the checkpoint, and the context a step hands to
the parts.  No part knows which model it is in; it sees its own parameters, its own tensors, the
step's token metadata and (for a mixer) its own cache entry and state.

Interfaces
----------
norm        ``tensors(params, prefix)``; ``__init__(params, prefix, weights, rt)``;
            ``forward(x, out=None)``; ``add_forward(x, delta, rows=None)`` -> normed rows, with
            ``x += delta`` written back (fused residual add, ``kernels/rmsnorm.py:21-39``).
            Optional: ``rms_params() -> (weight, eps)`` declares the plain RMS arithmetic, which lets the
            decode products fold the norm into themselves (``fused_rms`` below).
position    ``__init__(params, head_dim, rt)``; gives ``rotary_dim`` and ``inv_freq`` to the mixer.
mixer       ``tensors``; ``__init__``; ``kv_need()`` / ``state_need()``;
            ``forward(h, ctx, cache, state, owns_cache)`` -> ``[tokens, hidden]`` (not yet added).
ffn         ``tensors``; ``__init__``; ``forward(h, ctx)`` -> ``[tokens, hidden]``.
block       ``__init__(norm_mixer, mixer, norm_ffn, ffn)`` (``norm_ffn`` and ``ffn`` are None in a layer without a
            feed-forward; a layer that lists extra parts also passes ``extra={name: part}``);
            ``forward(res, ctx, cache, state, owns_cache)`` -> ``Residual``: the stream, plus either the
            not-yet-added output of the block's last part (so the next norm can fuse the add) or the
            stream's sums of squares (so the next fused product can normalise it).
Optional, for few rows (decode): a mixer or feed-forward may offer
            ``forward_normed(x, ss, ss_parts, norm, ...) -> (ss, ss_parts)``: it normalises ``x`` itself
            inside its first product, adds its output into ``x`` in place inside its last product, and
            returns the new sums of squares; ``can_fuse(n_rows, norm)`` says when.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Mapping, NamedTuple, Optional, Tuple

import torch

from ..config.spec import PartSpec


class TensorInfo(NamedTuple):
    """One checkpoint tensor a part expects.  ``kind``: "matrix" (a product's weight), "vector"
    (norm weights and other 1-D tensors, kept in 32-bit on the device) or "table" (embedding)."""

    shape: Tuple[int, ...]
    kind: str
    optional: bool = False


@dataclass
class Runtime:
    """Where and how the parts compute."""

    dtype: torch.dtype           # activation dtype: torch.float32 or torch.bfloat16
    device: torch.device
    page_size: int = 64
    sm_count: int = 148
    small_m_max: int = 16         # decode rows up to which weights stream through registers into mma.sync (csrc/gemm_decode.cu)
    stream_m_max: int = 0        # decode rows up to which the tcgen05 weight-streaming product runs above that (0: the library's)
    ffn_chunk_rows: int = 16384  # rows of the feed-forward processed at once (bounds [rows, 2I])
    fuse_decode: bool = True     # few rows: fold norms, residual adds and SiLU*mul into the products
    pdl: bool = True             # launch the fused decode products as programmatic dependents
    norm_ahead: bool = False     # fused decode: a residual product leaves the stream weighted for the next norm (one rounding fewer than the reference)
    tcgen05: bool = True         # prompts: attention on tcgen05.mma / tensor memory / TMA where sizes allow

    @property
    def is_bf16(self) -> bool:
        return self.dtype == torch.bfloat16


@dataclass
class StepContext:
    """Token metadata of one step, on the device unless noted."""

    n_tokens: int                 # activation rows (padding rows included)
    n_seqs: int
    tokens: torch.Tensor          # int32 [n_tokens]
    cu_q: torch.Tensor            # int32 [n_seqs + 1]: sequence b's tokens are cu_q[b]..cu_q[b+1]-1
    seq_slot: torch.Tensor        # int32 [n_seqs]: cache slot, -1 for a padding sequence
    tok_slot: torch.Tensor        # int32 [n_tokens]
    tok_pos: torch.Tensor         # int32 [n_tokens]: absolute position of each token
    decode: bool                  # host: every sequence brings exactly one token
    max_kv: int = 0               # host: no sequence is longer than this after the step (a bound, may be loose)
    tile_tok0: Optional[torch.Tensor] = None   # int32 [n_tiles]: first packed token of a query tile
    tile_rows: Optional[torch.Tensor] = None   # int32 [n_tiles]: tokens in the tile (<= tile_size)
    n_tiles: int = 0
    tile_size: int = 0
    extras: Dict[str, Any] = field(default_factory=dict)


@dataclass
class Residual:
    """The residual stream between blocks.  ``delta`` is the previous part's output that has not
    been added to ``x`` yet (the next norm fuses the add).  ``ss`` holds per-row sums of squares of
    ``x`` in ``ss_parts`` blocks of 64 floats, as the fused decode products leave them for the next
    norm; it is only meaningful while ``delta`` is None."""

    x: torch.Tensor
    delta: Optional[torch.Tensor] = None
    ss: Optional[torch.Tensor] = None
    ss_parts: int = 0
    # ``x`` already multiplied by the weight of the norm ``xw_norm`` (and rounded): left by a fused decode
    # product for the product behind that norm, which then has no prologue (it scales its sums instead)
    xw: Optional[torch.Tensor] = None
    xw_norm: Optional[Any] = None


def fused_rms(norm) -> Optional[Tuple[torch.Tensor, float]]:
    """``(weight, eps)`` if ``norm`` declares, through a method ``rms_params()``, that it computes exactly
    ``weight * cast(x32 * rsqrt(mean(x32^2) + eps))`` with a 32-bit ``weight`` -- the arithmetic the fused decode
    products fold into themselves -- else None.  A norm of any other arithmetic (a ``1 + w`` weight, a bias, a
    mean subtracted) simply does not offer the method, whatever its class is called, and is run as its own kernel."""
    get = getattr(norm, "rms_params", None)
    if not callable(get):
        return None
    params = get()
    if params is None:
        return None
    weight, eps = params
    if not isinstance(weight, torch.Tensor) or weight.dtype != torch.float32 or weight.dim() != 1:
        return None
    return weight, float(eps)


class Registry:
    def __init__(self, what: str):
        self.what = what
        self._classes: Dict[str, Any] = {}

    def register(self, kind: str, cls: Any = None):
        """``register(kind, cls)`` or ``@register(kind)``."""
        if cls is None:
            def deco(c):
                self._classes[kind] = c
                return c
            return deco
        self._classes[kind] = cls
        return cls

    def unregister(self, kind: str) -> None:
        self._classes.pop(kind, None)

    def get(self, kind: str) -> Any:
        if kind not in self._classes:
            raise KeyError(f"unknown {self.what} kind {kind!r}; registered: " + ", ".join(sorted(self._classes)))
        return self._classes[kind]

    def kinds(self):
        return sorted(self._classes)


MIXERS = Registry("mixer")
FFNS = Registry("feed-forward")
NORMS = Registry("norm")
POSITIONS = Registry("position encoding")
BLOCKS = Registry("block arrangement")
EMBEDDINGS = Registry("embedding")
HEADS = Registry("output head")

FAMILIES = {"mixer": MIXERS, "ffn": FFNS, "norm": NORMS}   # the registries a layer's extra parts are built from

register_mixer = MIXERS.register
register_ffn = FFNS.register
register_norm = NORMS.register
register_position = POSITIONS.register
register_block = BLOCKS.register
register_embedding = EMBEDDINGS.register
register_head = HEADS.register
