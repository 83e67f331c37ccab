"""Configuration and registry (no GPU)."""
import copy
import json

import pytest

from kipp_b200.config import (ConfigError, Qwen3Config, config_from_dict, get_architecture,
                              load_config, register_architecture, registered_architectures,
                              unregister_architecture)
from kipp_b200.config.base import ModelConfig
from tiny import TINY_A, TINY_B, TINY_C


def test_reads_every_size_from_json():
    a, b = config_from_dict(TINY_A), config_from_dict(TINY_B)
    assert isinstance(a, Qwen3Config)
    for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                "num_attention_heads", "num_key_value_heads", "head_dim", "max_position_embeddings",
                "rope_theta", "rms_norm_eps", "tie_word_embeddings"):
        assert getattr(a, key) == TINY_A[key]
        assert getattr(b, key) == TINY_B[key]
        assert getattr(a, key) != getattr(b, key), key       # the two differ in every size
    assert (a.q_dim, a.kv_dim, a.group_size) == (64, 32, 2)
    assert (b.q_dim, b.kv_dim, b.group_size) == (256, 32, 8)     # q width != hidden
    assert b.q_dim != b.hidden_size


def test_head_dim_default_and_roundtrip(tmp_path):
    cfg = copy.deepcopy(TINY_A)
    del cfg["head_dim"]
    c = config_from_dict(cfg)
    assert c.head_dim == 16
    c.save(str(tmp_path))
    again = load_config(str(tmp_path))
    assert again == c
    assert json.load(open(tmp_path / "config.json"))["architectures"] == ["Qwen3ForCausalLM"]


def test_window_layers():
    c = config_from_dict(TINY_C)
    assert [c.layer_window(i) for i in range(4)] == [None, 40, 40, None]
    cfg = dict(TINY_A, use_sliding_window=True, sliding_window=8, max_window_layers=1)
    c = config_from_dict(cfg)
    assert [c.layer_window(i) for i in range(2)] == [None, 8]
    assert config_from_dict(TINY_A).layer_window(1) is None


@pytest.mark.parametrize("change, word", [
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"attention_bias": True}, "bias"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, "rope_scaling"),
    ({"vocab_size": 0}, "positive"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
    ({"vocab_size": "many"}, "integer"),
    ({"tie_word_embeddings": 1}, "true or false"),
    ({"layer_types": ["full_attention"]}, "one entry per layer"),
    ({"use_sliding_window": True}, "sliding_window"),
])
def test_rejects(change, word):
    with pytest.raises(ConfigError, match=word):
        config_from_dict(dict(TINY_A, **change))


def test_missing_key_and_unknown_architecture(tmp_path):
    cfg = dict(TINY_A)
    del cfg["rope_theta"]
    with pytest.raises(ConfigError, match="rope_theta"):
        config_from_dict(cfg)
    with pytest.raises(ConfigError, match="unsupported architecture"):
        config_from_dict(dict(TINY_A, architectures=["LlamaForCausalLM"]))
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict({"vocab_size": 3})
    with pytest.raises(ConfigError, match="no config.json"):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        load_config(str(tmp_path))


def test_registry_takes_another_architecture():
    import dataclasses

    @dataclasses.dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        width: int = 4

    register_architecture("ToyForTests", ToyConfig, lambda c: ("built", c.width))
    try:
        assert "ToyForTests" in registered_architectures()
        c = config_from_dict({"architectures": ["ToyForTests"], "width": 7})
        assert get_architecture("ToyForTests").build(c) == ("built", 7)
        with pytest.raises(ValueError):
            register_architecture("ToyForTests", ToyConfig, lambda c: None)
    finally:
        unregister_architecture("ToyForTests")
    assert "Qwen3ForCausalLM" in registered_architectures()


def test_presets_are_data_and_valid():
    """Every preset file parses into a valid typed configuration; the benchmark
    preset has the sizes of the 4B benchmark configuration."""
    from kipp_b200.config import config_from_dict, load_preset, preset_names
    names = preset_names()
    assert {"tiny-a", "tiny-b", "qwen3-4b", "qwen3-8b", "qwen3-32b"} <= set(names)
    for name in names:
        cfg_dict, init = load_preset(name)
        cfg = config_from_dict(cfg_dict)
        assert cfg.num_attention_heads % cfg.num_key_value_heads == 0
        assert init["seed"] >= 0 and init["sigma"] > 0
    cfg = config_from_dict(load_preset("qwen3-4b")[0])
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads,
            cfg.head_dim, cfg.intermediate_size, cfg.vocab_size) == (36, 2560, 32, 8, 128, 9728, 151936)
    assert cfg.tie_word_embeddings and load_preset("qwen3-4b")[1]["seed"] == 2
    with pytest.raises(KeyError):
        load_preset("no-such-model")
