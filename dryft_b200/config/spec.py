"""Architecture-neutral description of a decoder: which parts each layer is made
of, with every size and constant as a parameter, and the order the layers run in.

A ``ModelSpec`` is plain data.  An architecture's typed configuration turns its
``config.json`` into one (``Qwen3Config.model_spec``); the model builder
(``dryft_b200.engine.model.build_model``) turns the spec into parts by looking
each ``PartSpec.kind`` up in the part registries.  Nothing below this file knows
which architecture it serves.

The reference engine hard-codes one layer shape (``engine/dryft_qwen3/model.py:152-184``)
and one weight list (``engine/dryft_qwen3/weights.py:90-113``); here both are data.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part: ``kind`` names a registered class, ``params`` are its sizes and constants."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class ExtraPart:
    """A part of a layer beyond the usual four: ``family`` says which registry builds it ("norm", "ffn" or
    "mixer"), ``name`` is what the block arrangement knows it by (a norm behind the mixer's output, say)."""

    name: str
    family: str
    spec: PartSpec
    prefix: str


@dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement (``block``) of a mixer, a feed-forward and their norms.

    The ``*_prefix`` fields are the checkpoint name prefixes of the four parts
    (``model.layers.3.self_attn.``); each part appends its own local tensor names
    (``q_proj.weight``), so no part carries an architecture's naming.  A layer without a feed-forward
    leaves ``ffn`` and ``norm_ffn`` ``None``; a layer with more parts (norms on both sides of a part, a
    second feed-forward) lists them in ``extra``, and its block arrangement is handed them by name.
    """

    block: str
    mixer: PartSpec
    ffn: Optional[PartSpec]
    norm_mixer: PartSpec
    norm_ffn: Optional[PartSpec]
    mixer_prefix: str
    ffn_prefix: str
    norm_mixer_prefix: str
    norm_ffn_prefix: str
    extra: Tuple[ExtraPart, ...] = ()


@dataclass(frozen=True)
class RunStep:
    """One entry of the run order.

    ``layer`` indexes ``ModelSpec.layers`` and may occur more than once (the
    weights are then shared; every occurrence still owns a cache entry unless it
    borrows one).  ``cache_from`` is the index of an *earlier* run step whose
    cache entry this step reads instead of owning one.
    """

    layer: int
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[RunStep, ...]
    final_norm: PartSpec
    head: PartSpec
    embedding_prefix: str = "model.embed_tokens."
    final_norm_prefix: str = "model.norm."
    head_prefix: str = "lm_head."

    def validate(self) -> None:
        if not self.layers:
            raise ValueError("model spec has no layers")
        if not self.schedule:
            raise ValueError("model spec has an empty run order")
        for i, layer in enumerate(self.layers):
            if (layer.ffn is None) != (layer.norm_ffn is None):
                raise ValueError(f"layer {i}: a feed-forward and its norm go together (one of them is missing)")
            names = [e.name for e in layer.extra]
            if len(set(names)) != len(names):
                raise ValueError(f"layer {i}: two extra parts share a name: {names}")
            for e in layer.extra:
                if e.family not in ("norm", "ffn", "mixer"):
                    raise ValueError(f"layer {i}: extra part {e.name!r} has family {e.family!r}; known: norm, ffn, mixer")
        for i, st in enumerate(self.schedule):
            if not 0 <= st.layer < len(self.layers):
                raise ValueError(f"run step {i} names layer {st.layer}, but there are {len(self.layers)} layers")
            if st.cache_from is not None:
                if not 0 <= st.cache_from < i:
                    raise ValueError(f"run step {i} borrows the cache of step {st.cache_from}, which does not run before it")
                if self.schedule[st.cache_from].cache_from is not None:
                    raise ValueError(f"run step {i} borrows from step {st.cache_from}, which itself borrows a cache")
