"""The tensors a model spec expects to find in a checkpoint, asked of the parts themselves."""

from __future__ import annotations

from typing import Dict

from ..config.spec import ModelSpec
from ..parts.base import EMBEDDINGS, FAMILIES, FFNS, HEADS, MIXERS, NORMS, TensorInfo


def expected_tensors(spec: ModelSpec) -> Dict[str, TensorInfo]:
    out: Dict[str, TensorInfo] = {}

    def add(d: Dict[str, TensorInfo]) -> None:
        for k, v in d.items():
            if k in out and out[k].shape != v.shape:
                raise ValueError(f"two parts expect tensor {k} with different shapes: {out[k].shape} and {v.shape}")
            out[k] = v

    add(EMBEDDINGS.get(spec.embedding.kind).tensors(spec.embedding.params, spec.embedding_prefix))
    for layer in spec.layers:
        add(NORMS.get(layer.norm_mixer.kind).tensors(layer.norm_mixer.params, layer.norm_mixer_prefix))
        add(MIXERS.get(layer.mixer.kind).tensors(layer.mixer.params, layer.mixer_prefix))
        if layer.ffn is not None:
            add(NORMS.get(layer.norm_ffn.kind).tensors(layer.norm_ffn.params, layer.norm_ffn_prefix))
            add(FFNS.get(layer.ffn.kind).tensors(layer.ffn.params, layer.ffn_prefix))
        for e in layer.extra:
            add(FAMILIES[e.family].get(e.spec.kind).tensors(e.spec.params, e.prefix))
    add(NORMS.get(spec.final_norm.kind).tensors(spec.final_norm.params, spec.final_norm_prefix))
    add(HEADS.get(spec.head.kind).tensors(spec.head.params, spec.head_prefix))
    return out
