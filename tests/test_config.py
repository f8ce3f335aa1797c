"""Configuration: what config.json keys become, what is refused, and the registry."""

import json

import pytest

from conftest import TINY_A, TINY_B, TINY_C, TINY_E
from qwen3_from_scratch_b200.config import ConfigError, Qwen3Config
from qwen3_from_scratch_b200.registry import (build_model_spec, config_from_dict, load_config,
                                              registered_architectures)


def test_reads_every_size_from_the_file():
    cfg = config_from_dict(TINY_B)
    assert isinstance(cfg, Qwen3Config)
    assert (cfg.vocab_size, cfg.hidden_size, cfg.num_hidden_layers) == (384, 80, 3)
    assert (cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim) == (6, 2, 32)
    assert cfg.intermediate_size == 200 and cfg.rms_norm_eps == 1e-5 and cfg.rope_theta == 1e6
    assert cfg.tie_word_embeddings is False and cfg.max_position_embeddings == 256


def test_head_dim_defaults_to_width_over_heads_only_when_absent():
    data = dict(TINY_A)
    del data["head_dim"]
    assert config_from_dict(data).head_dim == 16
    data["head_dim"] = 32  # decoupled from hidden_size / heads, as in Qwen3
    assert config_from_dict(data).head_dim == 32


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "hidden_act", "num_hidden_layers",
                                 "max_position_embeddings", "num_key_value_heads", "num_attention_heads",
                                 "intermediate_size", "rms_norm_eps", "rope_theta"])
def test_missing_required_key_is_named(key):
    data = dict(TINY_A)
    del data[key]
    with pytest.raises(ConfigError, match=key):
        config_from_dict(data)


@pytest.mark.parametrize("patch, word", [
    ({"attention_bias": True}, "attention_bias"),
    ({"rope_scaling": {"type": "yarn", "factor": 4.0}}, "rope_scaling"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"vocab_size": "many"}, "vocab_size"),
    ({"num_hidden_layers": 0}, "num_hidden_layers"),
    ({"layer_types": ["full_attention"]}, "layer_types"),
    ({"layer_types": ["full_attention", "linear_attention"]}, "linear_attention"),
    ({"layer_types": ["sliding_attention", "full_attention"]}, "sliding_window"),
    ({"sliding_window": -4}, "sliding_window"),
])
def test_unsupported_values_are_refused(patch, word):
    data = dict(TINY_A)
    data.update(patch)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(data)


def test_window_layers_from_either_form_of_the_keys():
    b = config_from_dict(TINY_E)  # use_sliding_window + max_window_layers
    assert b.layer_types == ("full_attention", "sliding_attention", "sliding_attention")
    assert b.sliding_window == 24
    c = config_from_dict(TINY_C)  # explicit layer_types
    assert c.layer_types == ("sliding_attention", "full_attention") and c.sliding_window == 40
    off = dict(TINY_E, use_sliding_window=False)
    assert config_from_dict(off).sliding_window is None
    assert set(config_from_dict(off).layer_types) == {"full_attention"}


def test_unknown_architecture_lists_the_registered_ones():
    data = dict(TINY_A, architectures=["LlamaForCausalLM"])
    with pytest.raises(ConfigError, match="Qwen3ForCausalLM"):
        config_from_dict(data)
    assert "Qwen3ForCausalLM" in registered_architectures()


def test_round_trip_through_a_folder(tmp_path):
    for data in (TINY_A, TINY_B, TINY_C, TINY_E):
        cfg = config_from_dict(data)
        cfg.save(str(tmp_path))
        assert load_config(str(tmp_path)) == cfg
        assert json.load(open(tmp_path / "config.json"))["architectures"] == ["Qwen3ForCausalLM"]


def test_spec_takes_every_constant_from_the_configuration():
    spec = build_model_spec(config_from_dict(TINY_C))
    assert len(spec.layers) == 2 and [c.layer for c in spec.order] == [0, 1]
    name, block = spec.layers[0]
    mixer = block.params["mixer"]
    assert name == "model.layers.0" and mixer.kind == "gqa_attention"
    assert mixer.params["window"] == 40 and spec.layers[1][1].params["mixer"].params["window"] is None
    assert mixer.params["num_heads"] == 5 and mixer.params["num_kv_heads"] == 1 and mixer.params["head_dim"] == 48
    assert mixer.params["position"].params["theta"] == 50000.0
    assert block.params["norm1"].params == {"dim": 96, "eps": 1e-6}
    assert spec.head[1].params["tied_to"] is None and spec.vocab_size == 331
    tied = build_model_spec(config_from_dict(TINY_A))
    assert tied.head[1].params["tied_to"] == "model.embed_tokens.weight"
    assert "lm_head.weight" in tied.ignorable_weights


def test_bad_json_and_missing_file(tmp_path):
    with pytest.raises(ConfigError, match="no config.json"):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        load_config(str(tmp_path))
