"""Weights: the random-weights mode writes a model folder that loads back by tensor name; a
checkpoint that does not match is refused with ONE error listing every missing tensor, every
unexpected tensor and every wrong shape; precision rules on the way to the device."""

import json
import os

import pytest
import torch
from safetensors.torch import load_file, save_file

import helpers as H
from dryft_b200.config import config_from_dict
from dryft_b200.weights import (Checkpoint, CheckpointSource, WeightsError, expected_tensors, random_state_dict,
                                resolve_dtype, write_random_model)


def _spec(name):
    return config_from_dict(H.config_dict(name)).model_spec()


def test_random_model_folder_roundtrip(tmp_path):
    d = H.make_model_dir("b", str(tmp_path / "m"))
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    raw = json.load(open(os.path.join(d, "config.json")))
    assert raw["architectures"] == ["Qwen3ForCausalLM"] and raw["vocab_size"] == 384
    ck = Checkpoint(d)
    exp = expected_tensors(_spec("b"))
    ck.check(exp)
    names = set(ck.names())
    # Hugging Face tensor names (engine/dryft_qwen3/weights.py:81-114)
    for n in ("model.embed_tokens.weight", "model.norm.weight", "lm_head.weight", "model.layers.2.self_attn.q_proj.weight",
              "model.layers.0.self_attn.k_norm.weight", "model.layers.1.mlp.gate_proj.weight",
              "model.layers.1.post_attention_layernorm.weight", "model.layers.0.input_layernorm.weight"):
        assert n in names
    assert len(names) == 2 + 1 + 3 * 11
    t = load_file(os.path.join(d, "model.safetensors"))
    assert all(v.dtype == torch.bfloat16 for v in t.values())
    assert abs(float(t["model.norm.weight"].float().mean()) - 1.0) < 0.1  # 1 + normal
    assert abs(float(t["model.layers.0.mlp.up_proj.weight"].float().std()) - H.STD) < 0.01
    # same seed, same bytes; other seed, other values
    d2 = H.make_model_dir("b", str(tmp_path / "m2"))
    t2 = load_file(os.path.join(d2, "model.safetensors"))
    assert all(torch.equal(t[k], t2[k]) for k in t)
    other = random_state_dict(config_from_dict(H.config_dict("b")), seed=99)
    assert not torch.equal(other["model.norm.weight"], t["model.norm.weight"])
    # a tied model stores no lm_head
    da = H.make_model_dir("a", str(tmp_path / "a"))
    assert "lm_head.weight" not in Checkpoint(da).names()


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = H.make_model_dir("a", str(tmp_path / "m"))
    path = os.path.join(d, "model.safetensors")
    t = load_file(path)
    del t["model.layers.1.mlp.up_proj.weight"], t["model.norm.weight"]
    t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    t["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 32, dtype=torch.bfloat16)
    save_file(t, path)
    with pytest.raises(WeightsError) as e:
        Checkpoint(d).check(expected_tensors(_spec("a")))
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert [w[0] for w in err.wrong_shape] == ["model.layers.0.self_attn.q_proj.weight"]
    msg = str(err)
    for needle in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)", "expected (64, 64), found (64, 32)"):
        assert needle in msg


def test_untied_model_needs_lm_head_and_tied_one_may_omit_it(tmp_path):
    d = H.make_model_dir("b", str(tmp_path / "m"))
    path = os.path.join(d, "model.safetensors")
    t = load_file(path)
    del t["lm_head.weight"]
    save_file(t, path)
    with pytest.raises(WeightsError) as e:
        Checkpoint(d).check(expected_tensors(_spec("b")))
    assert e.value.missing == ["lm_head.weight"]
    da = H.make_model_dir("a", str(tmp_path / "a"))
    Checkpoint(da).check(expected_tensors(_spec("a")))  # tied: lm_head.weight is optional


def test_truncated_or_absent_file_is_a_clear_error(tmp_path):
    d = H.make_model_dir("a", str(tmp_path / "m"))
    path = os.path.join(d, "model.safetensors")
    data = open(path, "rb").read()
    open(path, "wb").write(data[: len(data) // 3])
    with pytest.raises(WeightsError) as e:
        Checkpoint(d)
    assert "model.safetensors" in str(e.value)
    os.remove(path)
    with pytest.raises(FileNotFoundError):
        Checkpoint(d)


def test_sharded_checkpoint_with_index(tmp_path):
    d = H.make_model_dir("a", str(tmp_path / "m"))
    t = load_file(os.path.join(d, "model.safetensors"))
    os.remove(os.path.join(d, "model.safetensors"))
    names = sorted(t)
    half = len(names) // 2
    parts = {"model-00001-of-00002.safetensors": names[:half], "model-00002-of-00002.safetensors": names[half:]}
    weight_map = {}
    for fn, ns in parts.items():
        save_file({n: t[n] for n in ns}, os.path.join(d, fn))
        weight_map.update({n: fn for n in ns})
    json.dump({"weight_map": weight_map}, open(os.path.join(d, "model.safetensors.index.json"), "w"))
    ck = Checkpoint(d)
    ck.check(expected_tensors(_spec("a")))
    assert torch.equal(ck.read(names[-1]), t[names[-1]])


def test_precision_rules():
    bf, f32, f16 = torch.bfloat16, torch.float32, torch.float16
    assert resolve_dtype(bf, bf, "matrix") == bf
    assert resolve_dtype(f32, bf, "matrix") == f32      # stored in 32-bit: stays so
    assert resolve_dtype(f16, bf, "table") == bf
    assert resolve_dtype(bf, bf, "vector") == f32       # norm weights: exact widening
    assert resolve_dtype(bf, f32, "matrix") == f32      # the 32-bit path widens everything
    assert resolve_dtype(torch.int64, bf, "table") == torch.int32


def test_source_loads_and_fuses_on_the_cpu(tmp_path):
    d = H.make_model_dir("b", str(tmp_path / "m"))
    ck = Checkpoint(d)
    src = CheckpointSource(ck, torch.bfloat16, torch.device("cpu"))
    p = "model.layers.1.self_attn."
    fused = src.load_fused([p + "q_proj.weight", p + "k_proj.weight", p + "v_proj.weight"], [192, 96, 96], 80)
    t = load_file(os.path.join(d, "model.safetensors"))
    assert fused.dtype == torch.bfloat16 and fused.shape == (384, 80)
    assert torch.equal(fused[:192], t[p + "q_proj.weight"]) and torch.equal(fused[288:], t[p + "v_proj.weight"])
    w = src.load("model.norm.weight", "vector")
    assert w.dtype == torch.float32 and torch.equal(w, t["model.norm.weight"].float())
    src32 = CheckpointSource(ck, torch.float32, torch.device("cpu"))
    assert src32.load(p + "o_proj.weight", "matrix").dtype == torch.float32
    # a model folder stored in 32-bit stays 32-bit in the bfloat16 path
    d32 = H.make_model_dir("a", str(tmp_path / "m32"), dtype=torch.float32)
    s = CheckpointSource(Checkpoint(d32), torch.bfloat16, torch.device("cpu"))
    assert s.load("model.embed_tokens.weight", "table").dtype == torch.float32
