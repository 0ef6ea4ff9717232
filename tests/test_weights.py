"""Weight loading errors and the random-weights mode (no GPU)."""
from __future__ import annotations

import json

import pytest
import torch
from safetensors.torch import load_file, save_file

from conftest import TINY_CONFIGS
from pylon_b200.config import Qwen3Config, read_config
from pylon_b200.models.decoder import DecoderModel
from pylon_b200.weights import Checkpoint, WeightError, write_random_model


def model_for(folder):
    architecture, config = read_config(folder)
    return DecoderModel(architecture.build_spec(config, 64))


def test_random_mode_writes_a_loadable_folder(tmp_path):
    config = Qwen3Config(**TINY_CONFIGS["tinyB"])
    write_random_model(config, 5, tmp_path)
    model = model_for(tmp_path)
    checkpoint = Checkpoint(tmp_path)
    checkpoint.verify(model.tensor_decls(), model.spec.ignored_tensors)
    tensors = load_file(str(tmp_path / "model.safetensors"))
    assert set(tensors) == set(model.tensor_decls())
    assert all(t.dtype == torch.bfloat16 for t in tensors.values())
    norm = tensors["model.layers.1.input_layernorm.weight"].float()
    matrix = tensors["model.layers.1.mlp.down_proj.weight"].float()
    assert abs(float(norm.mean()) - 1.0) < 0.02 and abs(float(matrix.mean())) < 0.002
    assert 0.015 < float(matrix.std()) < 0.025
    assert json.loads((tmp_path / "config.json").read_text())["architectures"] == ["Qwen3ForCausalLM"]


def test_same_seed_same_tensors_other_seed_other_tensors(tmp_path):
    config = Qwen3Config(**TINY_CONFIGS["tinyA"])
    a = load_file(str(write_random_model(config, 3, tmp_path / "a") / "model.safetensors"))
    b = load_file(str(write_random_model(config, 3, tmp_path / "b") / "model.safetensors"))
    c = load_file(str(write_random_model(config, 4, tmp_path / "c") / "model.safetensors"))
    assert all(torch.equal(a[name], b[name]) for name in a)
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])


def test_stored_32_bit_tensors_stay_32_bit(tmp_path):
    config = Qwen3Config(**TINY_CONFIGS["tinyA"])
    write_random_model(config, 0, tmp_path, dtype="float32")
    checkpoint = Checkpoint(tmp_path)
    assert checkpoint.fetch("model.norm.weight").dtype == torch.float32
    assert checkpoint.fetch("model.layers.0.self_attn.q_proj.weight").dtype == torch.float32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    config = Qwen3Config(**TINY_CONFIGS["tinyB"])
    write_random_model(config, 1, tmp_path)
    path = str(tmp_path / "model.safetensors")
    tensors = load_file(path)
    del tensors["model.layers.2.mlp.up_proj.weight"]
    del tensors["lm_head.weight"]
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)
    tensors["model.layers.1.self_attn.k_proj.weight"] = torch.zeros(96, 97, dtype=torch.bfloat16)
    save_file(tensors, path)
    model = model_for(tmp_path)
    with pytest.raises(WeightError) as caught:
        Checkpoint(tmp_path).verify(model.tensor_decls(), model.spec.ignored_tensors)
    error = caught.value
    assert error.missing == ["lm_head.weight", "model.layers.2.mlp.up_proj.weight"]
    assert error.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert error.wrong_shape == [("model.layers.1.self_attn.k_proj.weight", (96, 96), (96, 97))]
    text = str(error)
    for word in ("missing", "unexpected", "wrong shapes", "up_proj", "inv_freq", "(96, 97)"):
        assert word in text


def test_tied_model_tolerates_a_stored_head_and_untied_needs_it(tmp_path):
    tied = Qwen3Config(**TINY_CONFIGS["tinyA"])
    write_random_model(tied, 0, tmp_path)
    path = str(tmp_path / "model.safetensors")
    tensors = load_file(path)
    assert "lm_head.weight" not in tensors
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    save_file(tensors, path)
    model = model_for(tmp_path)
    Checkpoint(tmp_path).verify(model.tensor_decls(), model.spec.ignored_tensors)


def test_sharded_checkpoint(tmp_path):
    config = Qwen3Config(**TINY_CONFIGS["tinyA"])
    write_random_model(config, 0, tmp_path)
    tensors = load_file(str(tmp_path / "model.safetensors"))
    (tmp_path / "model.safetensors").unlink()
    names = sorted(tensors)
    halves = {"model-00001-of-00002.safetensors": names[: len(names) // 2], "model-00002-of-00002.safetensors": names[len(names) // 2 :]}
    weight_map = {}
    for file_name, members in halves.items():
        save_file({name: tensors[name] for name in members}, str(tmp_path / file_name))
        weight_map.update({name: file_name for name in members})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    model = model_for(tmp_path)
    checkpoint = Checkpoint(tmp_path)
    checkpoint.verify(model.tensor_decls(), model.spec.ignored_tensors)
    assert torch.equal(checkpoint.fetch(names[-1]), tensors[names[-1]])


def test_missing_folder_contents(tmp_path):
    with pytest.raises(FileNotFoundError):
        Checkpoint(tmp_path)
