"""Configuration: typed reading of config.json keys, errors that name the key, the registry."""
import copy
import json
import os

import pytest

import plain_llama as plain
from llm_infer_engine_b200.config import ConfigError, LlamaConfig, known_architectures, load_config
from llm_infer_engine_b200.config.spec import LayerCall
from llm_infer_engine_b200.models.llama import llama_spec


def test_reads_every_size_from_config_json():
    cfg = LlamaConfig.from_dict(plain.TINY_B)
    assert (cfg.hidden_size, cfg.num_hidden_layers, cfg.num_attention_heads, cfg.num_key_value_heads) == (96, 3, 3, 1)
    assert (cfg.head_dim, cfg.intermediate_size, cfg.vocab_size) == (32, 256, 384)
    assert cfg.rms_norm_eps == 1e-6 and cfg.rope_theta == 500000.0 and cfg.max_position_embeddings == 256
    assert cfg.rope_scaling.rope_type == "llama3" and cfg.rope_scaling.factor == 8.0
    assert cfg.rope_scaling.original_max_position_embeddings == 64
    assert cfg.tie_word_embeddings is False and cfg.eos_token_ids == (2, 3)
    a = LlamaConfig.from_dict(plain.TINY_A)
    assert a.rope_scaling is None and a.tie_word_embeddings is True and a.eos_token_ids == (2,)
    assert LlamaConfig.from_dict(a.to_dict()) == a


@pytest.mark.parametrize("key", ["hidden_size", "num_hidden_layers", "num_attention_heads", "intermediate_size",
                                 "vocab_size", "rms_norm_eps", "rope_theta", "max_position_embeddings"])
def test_missing_key_is_named(key):
    cfg = copy.deepcopy(plain.TINY_A)
    del cfg[key]
    with pytest.raises(ConfigError, match=key):
        LlamaConfig.from_dict(cfg)


def test_defaults_that_follow_from_other_keys():
    cfg = copy.deepcopy(plain.TINY_A)
    del cfg["num_key_value_heads"], cfg["head_dim"]
    c = LlamaConfig.from_dict(cfg)
    assert c.num_key_value_heads == 4 and c.head_dim == 16       # src/model.py:32: dim // n_heads


@pytest.mark.parametrize("key,value,match", [
    ("hidden_size", "64", "hidden_size"), ("vocab_size", -1, "vocab_size"), ("rms_norm_eps", "x", "rms_norm_eps"),
    ("num_key_value_heads", 3, "multiple"), ("hidden_act", "gelu", "hidden_act"), ("attention_bias", True, "attention_bias"),
    ("mlp_bias", True, "mlp_bias"), ("eos_token_id", 9999, "eos_token_id"), ("eos_token_id", "x", "eos_token_id"),
    ("head_dim", 15, "head_dim"), ("tie_word_embeddings", "yes", "tie_word_embeddings"),
])
def test_bad_values(key, value, match):
    cfg = copy.deepcopy(plain.TINY_A)
    cfg[key] = value
    with pytest.raises(ConfigError, match=match):
        LlamaConfig.from_dict(cfg)


def test_rope_scaling_errors_and_variants():
    cfg = copy.deepcopy(plain.TINY_B)
    cfg["rope_scaling"] = {"rope_type": "yarn", "factor": 2.0}
    with pytest.raises(ConfigError, match="yarn"):
        LlamaConfig.from_dict(cfg)
    cfg["rope_scaling"] = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0}
    with pytest.raises(ConfigError, match="original_max_position_embeddings"):
        LlamaConfig.from_dict(cfg)
    cfg["rope_scaling"] = {"type": "llama3", "factor": 8, "low_freq_factor": 1, "high_freq_factor": 4,
                           "original_max_position_embeddings": 64}      # legacy key, integers
    assert LlamaConfig.from_dict(cfg).rope_scaling.high_freq_factor == 4.0
    cfg["rope_scaling"] = {"rope_type": "default"}
    assert LlamaConfig.from_dict(cfg).rope_scaling is None
    # the newer single object
    del cfg["rope_scaling"], cfg["rope_theta"]
    cfg["rope_parameters"] = {"rope_theta": 12345.0, "rope_type": "llama3", "factor": 2.0, "low_freq_factor": 1.0,
                              "high_freq_factor": 3.0, "original_max_position_embeddings": 32}
    c = LlamaConfig.from_dict(cfg)
    assert c.rope_theta == 12345.0 and c.rope_scaling.factor == 2.0


def test_registry(tmp_path):
    assert "LlamaForCausalLM" in known_architectures()
    arch, cfg = load_config(plain.TINY_A)
    assert arch.name == "LlamaForCausalLM" and isinstance(cfg, LlamaConfig)
    bad = dict(plain.TINY_A, architectures=["NoSuchModel"])
    with pytest.raises(ConfigError, match="NoSuchModel.*LlamaForCausalLM"):
        load_config(bad)
    with pytest.raises(ConfigError, match="architectures"):
        load_config({k: v for k, v in plain.TINY_A.items() if k != "architectures"})
    with pytest.raises(ConfigError, match="config.json"):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="JSON"):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps(plain.TINY_B))
    assert load_config(str(tmp_path))[1].vocab_size == 384


def test_spec_is_data():
    spec = llama_spec(LlamaConfig.from_dict(plain.TINY_B))
    assert len(spec.layers) == 3 and [c.layer for c in spec.schedule] == [0, 1, 2]
    assert spec.layers[0].mixer.kind == "gqa_attention" and spec.layers[0].mixer.params["n_kv_heads"] == 1
    assert spec.layers[0].mixer.params["position"].params["scaling"]["factor"] == 8.0
    assert spec.final_norm.params["eps"] == 1e-6 and not spec.tie_head and tuple(spec.stop_token_ids) == (2, 3)
    spec.validate()
    import dataclasses
    with pytest.raises(ValueError, match="layer 7"):
        dataclasses.replace(spec, schedule=[LayerCall(7)]).validate()
    with pytest.raises(ValueError, match="earlier"):
        dataclasses.replace(spec, schedule=[LayerCall(0, cache_of=0)]).validate()
    dataclasses.replace(spec, schedule=[LayerCall(0), LayerCall(1, cache_of=0), LayerCall(0)]).validate()


def test_generation_config_adds_stop_ids(tmp_path):
    """Stop ids are the union of config.json's and generation_config.json's eos_token_id."""
    import json
    import plain_llama as plain
    from llm_infer_engine_b200.config import load_config
    (tmp_path / "config.json").write_text(json.dumps(dict(plain.TINY_A, eos_token_id=2)))
    arch, cfg = load_config(str(tmp_path))
    assert arch.to_spec(cfg).stop_token_ids == (2,)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [2, 7, 9], "temperature": 0.6}))
    arch, cfg = load_config(str(tmp_path))
    assert arch.to_spec(cfg).stop_token_ids == (2, 7, 9)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": "x"}))
    with pytest.raises(Exception, match="generation_config.json: eos_token_id"):
        load_config(str(tmp_path))
