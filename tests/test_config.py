"""Configuration: typed parsing of config.json keys, validation errors that name the key, the
architecture registry, and the model spec the configuration yields."""

import json

import pytest

from dryft_b200.config import (ConfigError, Qwen3Config, config_from_dict, known_architectures, load_config, preset,
                               register_architecture, unregister_architecture, PRESETS)
import helpers as H


def test_presets_parse_and_differ():
    a, b = config_from_dict(preset("tiny-a")), config_from_dict(preset("tiny-b"))
    for f in ("num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads", "head_dim",
              "intermediate_size", "vocab_size", "rms_norm_eps", "rope_theta", "tie_word_embeddings", "max_position_embeddings"):
        assert getattr(a, f) != getattr(b, f), f
    assert b.q_dim == 192 != b.hidden_size  # head size decoupled from the width
    big = config_from_dict(preset("qwen3-4b"))
    assert big.weight_bytes_per_decode_step(2) == 2 * (36 * ((4096 + 2048) * 2560 + 2560 * 4096 + 3 * 9728 * 2560) + 151936 * 2560)
    assert big.kv_bytes_per_token(2) == 147456  # engine/dryft_qwen3/config.py:103-105; AGENTS.md:183
    for name in PRESETS:
        config_from_dict(preset(name)).model_spec()


def test_head_dim_defaults_to_hidden_over_heads():
    raw = H.config_dict("a")
    del raw["head_dim"]
    assert config_from_dict(raw).head_dim == 64 // 4
    raw["head_dim"] = 0
    assert config_from_dict(raw).head_dim == 16


def test_rope_theta_may_sit_in_rope_parameters():
    raw = H.config_dict("a")
    theta = raw.pop("rope_theta")
    raw["rope_parameters"] = {"rope_type": "default", "rope_theta": theta}
    assert config_from_dict(raw).rope_theta == theta


@pytest.mark.parametrize("key,value,needle", [
    ("hidden_act", "gelu", "hidden_act"),
    ("attention_bias", True, "attention_bias"),
    ("rope_scaling", {"type": "yarn", "factor": 4}, "rope_scaling"),
    ("num_key_value_heads", 3, "num_key_value_heads"),
    ("head_dim", 15, "head_dim"),
    ("vocab_size", -1, "vocab_size"),
    ("rms_norm_eps", 0.0, "rms_norm_eps"),
    ("num_hidden_layers", 2.5, "num_hidden_layers"),
])
def test_bad_values_name_the_key(key, value, needle):
    raw = H.config_dict("a")
    raw[key] = value
    with pytest.raises(ConfigError) as e:
        config_from_dict(raw)
    assert needle in str(e.value)


def test_missing_keys_are_listed_together():
    raw = H.config_dict("a")
    del raw["vocab_size"], raw["rope_theta"], raw["intermediate_size"]
    with pytest.raises(ConfigError) as e:
        config_from_dict(raw)
    msg = str(e.value)
    assert "vocab_size" in msg and "rope_theta" in msg and "intermediate_size" in msg


def test_unknown_architecture_lists_known_ones(tmp_path):
    raw = H.config_dict("a")
    raw["architectures"] = ["LlamaForCausalLM"]
    with pytest.raises(KeyError) as e:
        config_from_dict(raw)
    assert "LlamaForCausalLM" in str(e.value) and "Qwen3ForCausalLM" in str(e.value)
    raw["architectures"] = []
    with pytest.raises(KeyError):
        config_from_dict(raw)
    with pytest.raises(FileNotFoundError):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps(H.config_dict("b")))
    assert isinstance(load_config(str(tmp_path)), Qwen3Config)


def test_registry_takes_new_architectures():
    class Other:
        def __init__(self, raw):
            self.raw = raw

    register_architecture("OtherForCausalLM", Other)
    try:
        assert "OtherForCausalLM" in known_architectures()
        assert isinstance(config_from_dict({"architectures": ["OtherForCausalLM"]}), Other)
    finally:
        unregister_architecture("OtherForCausalLM")
    assert "OtherForCausalLM" not in known_architectures()


def test_sliding_window_layer_types():
    c = config_from_dict(H.config_dict("c"))
    assert c.sliding_window == 40
    assert c.layer_types == ("full_attention", "sliding_attention", "sliding_attention", "sliding_attention")
    spec = c.model_spec()
    assert [l.mixer["window"] for l in spec.layers] == [None, 40, 40, 40]
    raw = H.config_dict("c")
    raw["layer_types"] = ["sliding_attention", "full_attention", "full_attention", "sliding_attention"]
    assert [l.mixer["window"] for l in config_from_dict(raw).model_spec().layers] == [40, None, None, 40]
    raw["layer_types"] = ["full_attention"] * 3
    with pytest.raises(ConfigError):
        config_from_dict(raw)
    raw = H.config_dict("c")
    del raw["sliding_window"]
    with pytest.raises(ConfigError):
        config_from_dict(raw)
    # use_sliding_window false: the other keys are ignored
    raw = H.config_dict("c")
    raw["use_sliding_window"] = False
    assert config_from_dict(raw).sliding_window is None


def test_model_spec_carries_every_constant_and_roundtrips():
    c = config_from_dict(H.config_dict("b"))
    spec = c.model_spec()
    assert len(spec.layers) == 3 and [s.layer for s in spec.schedule] == [0, 1, 2]
    m = spec.layers[1].mixer
    assert (m.kind, m["num_heads"], m["num_kv_heads"], m["head_dim"]) == ("attention", 6, 3, 32)
    assert m["scale"] == pytest.approx(32 ** -0.5) and m["qk_norm"]["eps"] == 1e-5 and m["position"]["theta"] == 1e6
    assert spec.layers[1].ffn["intermediate_size"] == 224 and spec.final_norm["eps"] == 1e-5
    assert spec.head["tied"] is False and spec.layers[2].mixer_prefix == "model.layers.2.self_attn."
    assert config_from_dict(c.to_dict()) == c
    c3 = config_from_dict(H.config_dict("c"))
    assert config_from_dict(c3.to_dict()) == c3


def test_run_order_is_validated():
    from dataclasses import replace

    from dryft_b200.config.spec import RunStep

    spec = config_from_dict(H.config_dict("a")).model_spec()
    replace(spec, schedule=(RunStep(0), RunStep(1), RunStep(0), RunStep(1, cache_from=1))).validate()
    with pytest.raises(ValueError):
        replace(spec, schedule=(RunStep(0), RunStep(5))).validate()
    with pytest.raises(ValueError):
        replace(spec, schedule=(RunStep(0, cache_from=0),)).validate()
    with pytest.raises(ValueError):
        replace(spec, schedule=(RunStep(0), RunStep(1, cache_from=0), RunStep(1, cache_from=1))).validate()


def test_layer_spec_checks_its_optional_and_extra_parts():
    from dryft_b200.config import ExtraPart, LayerSpec, ModelSpec, PartSpec, RunStep

    norm = PartSpec("rmsnorm", {"size": 8, "eps": 1e-6})
    mixer = PartSpec("attention", {})
    ffn = PartSpec("swiglu", {})

    def spec(layer):
        return ModelSpec("X", 10, 8, 16, PartSpec("embedding", {}), (layer,), (RunStep(0),), norm, PartSpec("lm_head", {}))

    spec(LayerSpec("prenorm", mixer, None, norm, None, "a.", "", "n.", "")).validate()             # no feed-forward
    spec(LayerSpec("prenorm", mixer, ffn, norm, norm, "a.", "f.", "n.", "m.",
                   extra=(ExtraPart("post", "norm", norm, "p."),))).validate()
    with pytest.raises(ValueError, match="go together"):
        spec(LayerSpec("prenorm", mixer, ffn, norm, None, "a.", "f.", "n.", "")).validate()
    with pytest.raises(ValueError, match="share a name"):
        spec(LayerSpec("prenorm", mixer, ffn, norm, norm, "a.", "f.", "n.", "m.",
                       extra=(ExtraPart("post", "norm", norm, "p."), ExtraPart("post", "norm", norm, "q.")))).validate()
    with pytest.raises(ValueError, match="family"):
        spec(LayerSpec("prenorm", mixer, ffn, norm, norm, "a.", "f.", "n.", "m.",
                       extra=(ExtraPart("post", "table", norm, "p."),))).validate()
