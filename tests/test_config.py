"""Configuration and registry (no GPU)."""
import json
import os

import pytest

from janas_b200.config import (ConfigError, ModelSpec, PartSpec, Qwen3Config, RunEntry,
                               config_from_dict, config_from_dir, known_architectures)
from tiny import TINY


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
def test_reads_every_key(name):
    d = TINY[name]
    c = config_from_dict(d)
    assert isinstance(c, Qwen3Config)
    for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                "num_attention_heads", "num_key_value_heads", "head_dim",
                "max_position_embeddings", "rms_norm_eps", "rope_theta", "tie_word_embeddings"):
        assert getattr(c, key) == d[key], key
    assert config_from_dict(c.to_dict()) == c


def test_defaults_follow_the_reference():
    d = dict(TINY["A"])
    del d["head_dim"], d["tie_word_embeddings"]
    c = config_from_dict(d)
    assert c.head_dim == d["hidden_size"] // d["num_attention_heads"]
    assert c.tie_word_embeddings is False


def test_window_layers():
    c = config_from_dict(TINY["C"])
    assert c.layer_types == ("full_attention", "full_attention", "sliding_attention",
                             "sliding_attention")
    spec = c.to_model_spec()
    assert [l.mixer.params["window"] for l in spec.layers] == [0, 0, 37, 37]
    d = dict(TINY["C"], layer_types=["sliding_attention", "full_attention"] * 2)
    assert [l.mixer.params["window"] for l in config_from_dict(d).to_model_spec().layers] \
        == [37, 0, 37, 0]


@pytest.mark.parametrize("change, word", [
    ({"hidden_size": None}, "missing hidden_size"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"attention_bias": True}, "attention_bias"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4}}, "rope_scaling"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rms_norm_eps": 0}, "rms_norm_eps"),
    ({"vocab_size": 2.5}, "whole number"),
    ({"use_sliding_window": True, "sliding_window": None}, "sliding_window"),
    ({"layer_types": ["full_attention"]}, "layer_types"),
])
def test_refuses(change, word):
    with pytest.raises(ConfigError, match=word):
        config_from_dict(dict(TINY["A"], **change))


def test_registry():
    assert "Qwen3ForCausalLM" in known_architectures()
    with pytest.raises(ConfigError, match="not supported"):
        config_from_dict(dict(TINY["A"], architectures=["LlamaForCausalLM"]))
    d = dict(TINY["A"])
    del d["architectures"]
    assert isinstance(config_from_dict(d), Qwen3Config)      # by model_type
    del d["model_type"]
    with pytest.raises(ConfigError, match="names no architecture"):
        config_from_dict(d)


def test_from_dir(tmp_path):
    with pytest.raises(ConfigError, match="no config.json"):
        config_from_dir(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not JSON"):
        config_from_dir(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps(TINY["B"]))
    assert config_from_dir(str(tmp_path)).hidden_size == 96


def test_run_order_is_checked():
    spec = config_from_dict(TINY["A"]).to_model_spec()
    kw = dict(architecture="x", hidden_size=64, vocab_size=256, max_positions=128,
              layers=spec.layers, final_norm=spec.final_norm, tie_embeddings=True)
    ModelSpec(run_order=(RunEntry(0), RunEntry(1), RunEntry(0), RunEntry(1, cache_of=1)),
              **kw).validate()
    with pytest.raises(ConfigError, match="names layer"):
        ModelSpec(run_order=(RunEntry(2),), **kw).validate()
    with pytest.raises(ConfigError, match="has not run"):
        ModelSpec(run_order=(RunEntry(0, cache_of=1), RunEntry(1)), **kw).validate()
    with pytest.raises(ConfigError, match="owns none"):
        ModelSpec(run_order=(RunEntry(0), RunEntry(1, cache_of=0), RunEntry(0, cache_of=1)),
                  **kw).validate()
