"""Configuration: typed reading of config.json keys, errors that name the key, the registry."""
import json

import pytest

from qwen_decoder_b200.config import (ConfigError, Qwen2Config, config_from_dict, describe_model,
                                      known_architectures, load_config, write_config_json)
from tiny_configs import TINY_A, TINY_B, TINY_C


def test_reads_every_key():
    c = Qwen2Config.from_dict(TINY_B)
    assert (c.hidden_size, c.intermediate_size, c.num_hidden_layers) == (128, 352, 3)
    assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (4, 1, 32)
    assert (c.vocab_size, c.max_position_embeddings) == (1000, 512)
    assert c.rope_theta == 1e6 and c.rms_norm_eps == 1e-5 and c.tie_word_embeddings is False
    assert c.group_size == 4 and c.kv_dim == 32 and c.q_dim == 128
    c = Qwen2Config.from_dict(TINY_C)
    assert c.head_dim == 48 and c.q_dim == 288 and c.rope_pairing == "adjacent"


def test_defaults_and_eos():
    d = dict(TINY_A)
    del d["num_key_value_heads"]
    del d["rope_pairing"]
    d["eos_token_id"] = [3, 5]
    c = Qwen2Config.from_dict(d)
    assert c.num_key_value_heads == 4 and c.eos_token_ids == (3, 5) and c.rope_pairing == "half"
    d["eos_token_id"] = 7
    assert Qwen2Config.from_dict(d).eos_token_ids == (7,)


@pytest.mark.parametrize("key", ["hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                                 "vocab_size", "max_position_embeddings", "rope_theta", "rms_norm_eps"])
def test_missing_key_is_named(key):
    d = dict(TINY_A)
    del d[key]
    with pytest.raises(ConfigError, match=key):
        Qwen2Config.from_dict(d)


@pytest.mark.parametrize("patch,word", [
    ({"hidden_size": "64"}, "hidden_size"), ({"num_key_value_heads": 3}, "num_key_value_heads"),
    ({"use_sliding_window": True}, "use_sliding_window"), ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"type": "yarn"}}, "rope_scaling"), ({"rms_norm_eps": 0}, "rms_norm_eps"),
    ({"head_dim": 15}, "head_dim"), ({"rope_pairing": "odd"}, "rope_pairing"),
    ({"architectures": []}, "architectures"), ({"tie_word_embeddings": 1}, "tie_word_embeddings"),
])
def test_bad_values(patch, word):
    with pytest.raises(ConfigError, match=word):
        Qwen2Config.from_dict(dict(TINY_A, **patch))


def test_registry_and_round_trip(tmp_path):
    assert "Qwen2ForCausalLM" in known_architectures()
    with pytest.raises(ConfigError, match="unknown architecture.*Qwen2ForCausalLM"):
        config_from_dict(dict(TINY_A, architectures=["NoSuchModel"]))
    c = config_from_dict(TINY_C)
    write_config_json(c, str(tmp_path))
    assert load_config(str(tmp_path)) == c
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        load_config(str(tmp_path))
    with pytest.raises(ConfigError, match="no config.json"):
        load_config(str(tmp_path / "nowhere"))


def test_model_description_follows_the_configuration():
    spec = describe_model(Qwen2Config.from_dict(TINY_B))
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    m = spec.layers[1].mixer
    assert m.name == "gq_attention" and m.params["num_kv_heads"] == 1 and m.params["head_dim"] == 32
    assert spec.layers[1].norms["input"].params["eps"] == 1e-5
    assert spec.positions["rope"].params["base"] == 1e6
    assert spec.lm_head_tensor == "lm_head.weight"
    assert describe_model(Qwen2Config.from_dict(TINY_A)).lm_head_tensor is None
