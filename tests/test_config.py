"""Configuration and registry (no GPU)."""
from __future__ import annotations

import json

import pytest

from conftest import TINY_CONFIGS
from pylon_b200.config import ConfigError, EngineConfig, Qwen3Config, read_config, register_architecture
from pylon_b200.config.registry import ARCHITECTURES
from pylon_b200.models.qwen3 import qwen3_spec


def hf_dict(**changes):
    data = Qwen3Config(**TINY_CONFIGS["tinyB"]).to_dict()
    data.update(changes)
    return data


def test_round_trip_and_derived_sizes():
    config = Qwen3Config(**TINY_CONFIGS["tinyB"])
    again = Qwen3Config.from_dict(config.to_dict())
    assert again == config
    assert config.q_size == 192 and config.kv_size == 96 and config.q_size != config.hidden_size


def test_head_dim_and_kv_heads_defaults():
    data = hf_dict()
    del data["head_dim"], data["num_key_value_heads"]
    config = Qwen3Config.from_dict(data)
    assert config.head_dim == 96 // 6 and config.num_key_value_heads == 6


@pytest.mark.parametrize("changes, word", [
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"attention_bias": True}, "attention_bias"),
    ({"rope_scaling": {"type": "yarn"}}, "rope_scaling"),
    ({"use_sliding_window": True}, "sliding_window"),
    ({"model_type": "llama"}, "model_type"),
    ({"sliding_window": 4096}, "sliding_window"),
    ({"num_key_value_heads": 4}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"vocab_size": 0}, "vocab_size"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
    ({"num_hidden_layers": True}, "num_hidden_layers"),
])
def test_refusals(changes, word):
    with pytest.raises(ConfigError, match=word):
        Qwen3Config.from_dict(hf_dict(**changes))


def test_missing_key_is_named():
    data = hf_dict()
    del data["rope_theta"]
    with pytest.raises(ConfigError, match="rope_theta"):
        Qwen3Config.from_dict(data)


def test_eos_forms():
    assert Qwen3Config.from_dict(hf_dict(eos_token_id=7)).eos_token_ids == (7,)
    assert Qwen3Config.from_dict(hf_dict(eos_token_id=[7, 9])).eos_token_ids == (7, 9)
    assert Qwen3Config.from_dict(hf_dict()).eos_token_ids == ()


def test_registry_lookup(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(hf_dict()))
    architecture, config = read_config(tmp_path)
    assert architecture.name == "Qwen3ForCausalLM" and isinstance(config, Qwen3Config)
    (tmp_path / "config.json").write_text(json.dumps(hf_dict(architectures=["LlamaForCausalLM"])))
    with pytest.raises(ConfigError, match="Qwen3ForCausalLM"):
        read_config(tmp_path)
    (tmp_path / "config.json").write_text("{")
    with pytest.raises(ConfigError, match="JSON"):
        read_config(tmp_path)


def test_another_architecture_can_be_registered(tmp_path):
    class OtherConfig(Qwen3Config):
        architecture = "OtherForCausalLM"
        model_type = "other"

    register_architecture("OtherForCausalLM", OtherConfig, qwen3_spec)
    try:
        (tmp_path / "config.json").write_text(json.dumps(hf_dict(architectures=["OtherForCausalLM"], model_type="other")))
        architecture, config = read_config(tmp_path)
        assert architecture.name == "OtherForCausalLM" and type(config) is OtherConfig
    finally:
        del ARCHITECTURES["OtherForCausalLM"]


def test_spec_is_data():
    config = Qwen3Config(**TINY_CONFIGS["tinyA"])
    spec = qwen3_spec(config, 128)
    assert spec.max_positions == 128 and len(spec.layers) == 2 and [run.layer for run in spec.order] == [0, 1]
    assert spec.lm_head_name is None and "lm_head.weight" in spec.ignored_tensors
    mixer = spec.layers[0].block.params["mixer"]
    assert mixer.kind == "gqa_attention" and mixer.params["n_kv_heads"] == 2 and mixer.params["qk_norm_eps"] == 1e-6
    assert mixer.params["position"].params["theta"] == 10_000.0
    untied = qwen3_spec(Qwen3Config(**TINY_CONFIGS["tinyB"]))
    assert untied.lm_head_name == "lm_head.weight" and untied.max_positions == 512


def test_engine_config_env_names_and_checks():
    config = EngineConfig.from_env({"PYLON_PREFILL_CHUNK_SIZE": "512", "PYLON_MAX_BATCH_SIZE": "4", "PYLON_CUDA_GRAPHS": "1", "PYLON_ADMIT_SKIP": "0"})
    assert (config.prefill_chunk_size, config.max_batch_size, config.cuda_graphs, config.admit_skip) == (512, 4, True, 0)
    assert EngineConfig.from_env({}).prefill_chunk_size == 2048 and EngineConfig.from_env({}).max_batch_size == 32
    with pytest.raises(ValueError, match="PYLON_CUDA_GRAPHS"):
        EngineConfig.from_env({"PYLON_CUDA_GRAPHS": "yes"})
    with pytest.raises(ValueError, match="prefill_chunk_size"):
        EngineConfig(prefill_chunk_size=0)
    with pytest.raises(ValueError, match="dtype"):
        EngineConfig(dtype="float16")
