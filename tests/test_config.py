"""Configuration parsing, validation and the architecture registry."""
import json

import pytest

from helpers import TINY_A, TINY_B
from stratakv_b200.config import ConfigError, EngineConfig, LlamaConfig, load_config, known_architectures


def test_reads_every_key():
    config = LlamaConfig.from_dict(TINY_B)
    assert (config.hidden_size, config.intermediate_size, config.num_hidden_layers) == (96, 256, 3)
    assert (config.num_attention_heads, config.num_key_value_heads, config.head_dim) == (6, 3, 16)
    assert config.vocab_size == 384 and config.rms_norm_eps == 1e-6 and config.rope_theta == 500000.0
    assert config.tie_word_embeddings and config.eos_token_ids == (5, 7)
    assert config.q_dim == 96 and config.kv_dim == 48 and config.group_size == 2


def test_defaults_follow_the_schema():
    raw = dict(TINY_A)
    del raw["num_key_value_heads"], raw["head_dim"]
    config = LlamaConfig.from_dict(raw)
    assert config.num_key_value_heads == 4 and config.head_dim == 16
    raw = dict(TINY_A, rope_parameters={"rope_type": "default", "rope_theta": 12345.0})
    del raw["rope_theta"]
    assert LlamaConfig.from_dict(raw).rope_theta == 12345.0


def test_round_trip(tmp_path):
    config = LlamaConfig.from_dict(TINY_A)
    (tmp_path / "config.json").write_text(config.to_json())
    arch, again = load_config(tmp_path)
    assert arch.name == "LlamaForCausalLM" and again == config


@pytest.mark.parametrize("change,message", [
    ({"num_key_value_heads": 3}, "multiple of num_key_value_heads"),
    ({"head_dim": 15}, "even"),
    ({"hidden_size": 0}, "positive"),
    ({"vocab_size": -1}, "positive"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"attention_bias": True}, "attention_bias"),
    ({"mlp_bias": True}, "mlp_bias"),
    ({"rope_scaling": {"type": "linear", "factor": 2.0}}, "rope_scaling"),
    ({"eos_token_id": 999}, "outside the vocabulary"),
    ({"hidden_size": "64"}, "must be an integer"),
    ({"tie_word_embeddings": 1}, "true or false"),
])
def test_rejects(change, message):
    with pytest.raises(ConfigError, match=message):
        LlamaConfig.from_dict(dict(TINY_A, **change))


def test_missing_key_is_named():
    raw = dict(TINY_A)
    del raw["intermediate_size"]
    with pytest.raises(ConfigError, match="intermediate_size"):
        LlamaConfig.from_dict(raw)


def test_unknown_architecture_lists_known(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(dict(TINY_A, architectures=["MambaForCausalLM"])))
    with pytest.raises(ConfigError, match="LlamaForCausalLM"):
        load_config(tmp_path)
    assert "LlamaForCausalLM" in known_architectures()


def test_no_config_file(tmp_path):
    with pytest.raises(ConfigError, match="no config.json"):
        load_config(tmp_path)


def test_engine_config():
    config = EngineConfig(max_tokens=130, dtype="float32")
    assert config.num_blocks == 3 and config.slots == 3
    with pytest.raises(ConfigError):
        EngineConfig(max_tokens=0)
    with pytest.raises(ConfigError):
        EngineConfig(max_tokens=64, dtype="float16")
    with pytest.raises(ConfigError):
        EngineConfig(max_tokens=64, block_size=24)


def test_spec_is_data_with_no_hidden_sizes():
    from stratakv_b200.config.registry import resolve_architecture
    for raw in (TINY_A, TINY_B):
        config = LlamaConfig.from_dict(raw)
        spec = resolve_architecture(config.architecture).build_spec(config)
        assert len(spec.layers) == config.num_hidden_layers == len(spec.schedule)
        layer = spec.layers[-1]
        assert layer.mixer.head_dim == config.head_dim and layer.mixer.position.theta == config.rope_theta
        assert layer.mixer_norm.eps == config.rms_norm_eps and layer.ffn.intermediate_size == config.intermediate_size
        assert spec.stop_token_ids == config.eos_token_ids
        assert (spec.head.weight == spec.embedding.weight) == config.tie_word_embeddings
