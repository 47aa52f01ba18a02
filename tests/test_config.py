import copy

import pytest

import tiny_configs
from distengine_b200.config import ConfigError, EngineConfig, LlamaConfig
from distengine_b200.registry import known_architectures, resolve

BASE = tiny_configs.TINY_A["config"]


def test_llama_config_reads_its_keys():
    arch, cfg = resolve(BASE)
    assert arch.name == "LlamaForCausalLM" and isinstance(cfg, LlamaConfig)
    assert (cfg.vocab_size, cfg.hidden_size, cfg.intermediate_size) == (256, 64, 176)
    assert (cfg.num_hidden_layers, cfg.num_attention_heads, cfg.num_key_value_heads) == (2, 4, 2)
    assert cfg.head_dim == 16 and cfg.rms_norm_eps == 1e-5 and cfg.rope_theta == 10000.0
    assert cfg.max_position_embeddings == 128 and cfg.tie_word_embeddings is False
    assert resolve(cfg.to_json())[1] == cfg


def test_nested_rope_and_given_head_dim():
    _, cfg = resolve(tiny_configs.TINY_C["config"])
    assert cfg.rope_theta == 25000.0 and cfg.head_dim == 48
    assert cfg.num_attention_heads * cfg.head_dim != cfg.hidden_size
    specs = cfg.layer_specs()
    assert len(specs) == 2 and specs[0].mixer.params["head_dim"] == 48
    assert specs[0].mixer.params["position"].params == {"rotary_dim": 48, "theta": 25000.0}
    assert specs[1].prefix("mixer") == "model.layers.1.self_attn."
    assert [e.layer for e in cfg.plan()] == [0, 1]


def test_kv_heads_default_to_heads():
    data = copy.deepcopy(BASE)
    del data["num_key_value_heads"]
    assert resolve(data)[1].num_key_value_heads == 4


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "intermediate_size",
                                 "num_hidden_layers", "num_attention_heads", "rms_norm_eps",
                                 "rope_theta", "max_position_embeddings"])
def test_missing_key_is_named(key):
    data = copy.deepcopy(BASE)
    del data[key]
    with pytest.raises(ConfigError, match=key):
        resolve(data)


@pytest.mark.parametrize("change,match", [
    ({"num_key_value_heads": 3}, "multiple"),
    ({"hidden_size": 66}, "multiple"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 8.0}}, "llama3"),
    ({"rope_parameters": {"rope_type": "yarn", "rope_theta": 1e4}}, "yarn"),
    ({"attention_bias": True}, "attention_bias"),
    ({"mlp_bias": True}, "mlp_bias"),
    ({"hidden_act": "gelu"}, "gelu"),
    ({"vocab_size": 0}, "vocab_size"),
    ({"vocab_size": "256"}, "vocab_size"),
    ({"head_dim": 15}, "even"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
    ({"tie_word_embeddings": "yes"}, "tie_word_embeddings"),
])
def test_unsupported_values_are_refused(change, match):
    data = copy.deepcopy(BASE)
    data.update(change)
    with pytest.raises(ConfigError, match=match):
        resolve(data)


def test_unknown_architecture_lists_known_ones():
    data = copy.deepcopy(BASE)
    data["architectures"] = ["MambaForCausalLM"]
    with pytest.raises(ConfigError, match="LlamaForCausalLM"):
        resolve(data)
    assert "LlamaForCausalLM" in known_architectures()
    with pytest.raises(ConfigError, match="architectures"):
        resolve({k: v for k, v in BASE.items() if k != "architectures"})


def test_engine_config():
    cfg = EngineConfig(dtype="fp32", block_size=8)
    import torch
    assert cfg.dtype == torch.float32
    with pytest.raises(ValueError):
        EngineConfig(dtype="float16")
    with pytest.raises(ValueError):
        EngineConfig(block_size=24)
    with pytest.raises(ValueError):
        EngineConfig(max_batch_tokens=0)
