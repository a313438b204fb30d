"""Configuration: reading the architecture's own keys, validation, the registry."""
import copy
import json
import math

import pytest

from helpers import TINY_A, TINY_B
from llmplayer_b200.config import (
    LlamaConfig, config_from_dict, known_architectures, load_config, register_architecture, unregister_architecture,
)
from llmplayer_b200.config.registry import ArchitectureConfig
from llmplayer_b200.errors import ConfigError


def test_reads_every_key():
    c = config_from_dict(TINY_B)
    assert isinstance(c, LlamaConfig)
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads) == (3, 96, 3, 1)
    assert (c.head_dim, c.intermediate_size, c.vocab_size) == (32, 320, 384)
    assert c.rope_theta == 500000.0 and c.rms_norm_eps == 1e-6 and c.tie_word_embeddings is False
    s = c.rope_scaling
    assert (s.factor, s.low_freq_factor, s.high_freq_factor, s.original_max_position) == (4.0, 1.0, 4.0, 64)
    assert c.max_positions() == 256


def test_defaults_are_derived_not_invented():
    raw = copy.deepcopy(TINY_A)
    del raw["head_dim"], raw["num_key_value_heads"], raw["tie_word_embeddings"]
    c = config_from_dict(raw)
    assert c.head_dim == 64 // 4 and c.num_key_value_heads == 4 and c.tie_word_embeddings is False


@pytest.mark.parametrize("key", ["num_hidden_layers", "hidden_size", "num_attention_heads", "intermediate_size",
                                 "vocab_size", "rope_theta", "rms_norm_eps", "max_position_embeddings"])
def test_missing_key_is_named(key):
    raw = copy.deepcopy(TINY_A)
    del raw[key]
    with pytest.raises(ConfigError, match=key):
        config_from_dict(raw)


@pytest.mark.parametrize("patch,needle", [
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"hidden_size": -4}, "positive"),
    ({"vocab_size": 0}, "positive"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "yarn"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 2.0}}, "low_freq_factor"),
    ({"attention_bias": True}, "attention_bias"),
    ({"num_hidden_layers": "2"}, "integer"),
    ({"eos_token_id": 999}, "vocabulary"),
])
def test_bad_values(patch, needle):
    raw = copy.deepcopy(TINY_A)
    raw.update(patch)
    with pytest.raises(ConfigError, match=needle):
        config_from_dict(raw)


def test_round_trip_and_file(tmp_path):
    c = config_from_dict(TINY_B)
    assert config_from_dict(c.to_dict()) == c
    (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
    assert load_config(str(tmp_path)) == c
    with pytest.raises(ConfigError, match="config.json"):
        load_config(str(tmp_path / "nowhere"))


def test_rope_parameters_block_is_understood():
    raw = copy.deepcopy(TINY_A)
    del raw["rope_theta"], raw["rope_scaling"]
    raw["rope_parameters"] = {"rope_type": "llama3", "rope_theta": 12345.0, "factor": 8.0, "low_freq_factor": 1.0,
                              "high_freq_factor": 4.0, "original_max_position_embeddings": 32}
    c = config_from_dict(raw)
    assert c.rope_theta == 12345.0 and c.rope_scaling.factor == 8.0


def test_eos_forms():
    raw = copy.deepcopy(TINY_A)
    raw["eos_token_id"] = [3, 7]
    assert config_from_dict(raw).stop_token_ids() == (3, 7)
    raw["eos_token_id"] = 5
    assert config_from_dict(raw).stop_token_ids() == (5,)


def test_registry_hit_and_miss():
    assert "LlamaForCausalLM" in known_architectures()
    with pytest.raises(ConfigError, match="Unknown architecture.*LlamaForCausalLM"):
        config_from_dict({"architectures": ["NoSuchModel"]})
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict({"hidden_size": 4})

    class Other(ArchitectureConfig):
        architecture = "OtherForTest"

        @classmethod
        def from_dict(cls, raw):
            return cls()

    register_architecture("OtherForTest", Other)
    try:
        assert isinstance(config_from_dict({"architectures": ["OtherForTest"]}), Other)
        with pytest.raises(ConfigError, match="already"):
            register_architecture("OtherForTest", LlamaConfig)
    finally:
        unregister_architecture("OtherForTest")


def test_layout_follows_the_configuration():
    c = config_from_dict(TINY_B)
    lay = c.layout()
    assert len(lay.layers) == 3 and [r.layer for r in lay.run_order()] == [0, 1, 2]
    att = lay.layers[1].mixer
    assert (att.num_heads, att.num_kv_heads, att.head_dim, att.window) == (3, 1, 32, None)
    assert att.scale == 1.0 / math.sqrt(32) and att.position.theta == 500000.0
    assert att.q == "model.layers.1.self_attn.q_proj.weight"
    assert lay.layers[2].ffn.intermediate_size == 320 and lay.layers[0].mixer_norm.eps == 1e-6
    assert lay.head.weight == "lm_head.weight"
    assert config_from_dict(TINY_A).layout().head.weight == "model.embed_tokens.weight"
