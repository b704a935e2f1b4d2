"""Configuration and registry (no GPU)."""
import json

import pytest

import tiny_configs
from kestrel_llm_b200.config import (ConfigError, Qwen3Config, known_architectures, load_config,
                                     register_architecture, resolve_architecture)


def test_keys_are_read_and_typed():
    c = Qwen3Config.from_dict(tiny_configs.B)
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads) == (3, 96, 6, 2)
    assert (c.head_dim, c.intermediate_size, c.vocab_size) == (32, 200, 509)
    assert c.rope_theta == 1e6 and c.rms_norm_eps == 1e-5 and c.qk_norm_eps == 1e-5
    assert c.attention_bias and not c.tie_word_embeddings
    assert c.q_size == 192 and c.kv_size == 64 and c.group_size == 3
    assert all(c.layer_window(i) == 0 for i in range(3))


def test_defaults_and_head_dim_rule():
    raw = dict(architectures=["Qwen3ForCausalLM"], hidden_size=64, num_hidden_layers=1, num_attention_heads=4,
               intermediate_size=8, vocab_size=10)
    c = Qwen3Config.from_dict(raw)
    assert c.head_dim == 16 and c.num_key_value_heads == 4
    assert c.rope_theta == 10000.0 and c.rms_norm_eps == 1e-6 and not c.tie_word_embeddings


def test_window_layers():
    c = Qwen3Config.from_dict(tiny_configs.C)
    assert [c.layer_window(i) for i in range(4)] == [0, 40, 40, 0]
    assert c.qk_norm_eps == 2e-5 and c.rms_norm_eps == 3e-6
    raw = dict(tiny_configs.C)
    del raw["layer_types"]
    raw["max_window_layers"] = 3
    c2 = Qwen3Config.from_dict(raw)
    assert [c2.layer_window(i) for i in range(4)] == [0, 0, 0, 40]


def test_round_trip_through_json():
    for raw, _ in tiny_configs.CONFIGS.values():
        c = Qwen3Config.from_dict(raw)
        assert Qwen3Config.from_dict(json.loads(json.dumps(c.to_json_dict()))) == c


@pytest.mark.parametrize("key", ["hidden_size", "num_hidden_layers", "num_attention_heads", "intermediate_size",
                                 "vocab_size"])
def test_required_keys(key):
    raw = dict(tiny_configs.A)
    del raw[key]
    with pytest.raises(ConfigError, match=key):
        Qwen3Config.from_dict(raw)


@pytest.mark.parametrize("patch,msg", [
    (dict(num_key_value_heads=3), "multiple"),
    (dict(head_dim=15), "even"),
    (dict(hidden_act="gelu"), "hidden_act"),
    (dict(rope_scaling={"rope_type": "yarn", "factor": 4.0}), "rope_scaling"),
    (dict(hidden_size="64"), "integer"),
    (dict(vocab_size=0), "positive"),
    (dict(eos_token_id=999), "vocabulary"),
    (dict(layer_types=["full_attention"]), "layer_types"),
])
def test_rejections(patch, msg):
    raw = dict(tiny_configs.A)
    raw.update(patch)
    with pytest.raises(ConfigError, match=msg):
        Qwen3Config.from_dict(raw)


def test_nested_text_config():
    raw = {"architectures": ["Qwen3ForCausalLM"], "text_config": {k: v for k, v in tiny_configs.A.items()
                                                                   if k != "architectures"}}
    assert Qwen3Config.from_dict(raw).hidden_size == 64


def test_registry(tmp_path):
    assert "Qwen3ForCausalLM" in known_architectures()
    with pytest.raises(ConfigError, match="not registered.*Qwen3ForCausalLM"):
        resolve_architecture("LlamaForCausalLM")
    (tmp_path / "config.json").write_text(json.dumps(tiny_configs.A))
    assert load_config(str(tmp_path)).vocab_size == 256
    (tmp_path / "config.json").write_text(json.dumps({k: v for k, v in tiny_configs.A.items() if k != "architectures"}))
    with pytest.raises(ConfigError, match="architectures"):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{ not json")
    with pytest.raises(ConfigError, match="not JSON"):
        load_config(str(tmp_path))
    register_architecture("ToyForTest", Qwen3Config, lambda *a: None)
    assert resolve_architecture("ToyForTest").config_class is Qwen3Config
