"""Shared fixtures: tiny Qwen3 configurations, model folders in temporary places, markers."""
from __future__ import annotations

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for entry in (str(ROOT), str(ROOT / "tests")):
    if entry not in sys.path:
        sys.path.insert(0, entry)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# Tiny configurations that differ in every size and option Qwen3 dense has: head counts
# and group size, head size, widths that are no power of two, layers, vocabulary, rope
# base, norm eps, tied or untied head.  tinyC has the head size (64) and page size (64) at
# which the TMA-fed decode attention and the tcgen05 prefill attention run, with a group of 3.
TINY_CONFIGS = {
    "tinyA": dict(vocab_size=256, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                  head_dim=16, intermediate_size=128, max_position_embeddings=512, rope_theta=10_000.0,
                  rms_norm_eps=1e-6, tie_word_embeddings=True),
    "tinyB": dict(vocab_size=320, hidden_size=96, num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=3,
                  head_dim=32, intermediate_size=224, max_position_embeddings=512, rope_theta=1_000_000.0,
                  rms_norm_eps=1e-5, tie_word_embeddings=False),
    "tinyC": dict(vocab_size=288, hidden_size=80, num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=2,
                  head_dim=64, intermediate_size=176, max_position_embeddings=512, rope_theta=50_000.0,
                  rms_norm_eps=1e-6, tie_word_embeddings=False),
}
TINY_SEEDS = {"tinyA": 0, "tinyB": 1, "tinyC": 2}
TINY_PAGE_SIZES = {"tinyA": 16, "tinyB": 8, "tinyC": 64}


@pytest.fixture(scope="session")
def tiny_folders(tmp_path_factory):
    """name -> model folder (config.json + model.safetensors) written by the random-weights mode."""
    from pylon_b200.config import Qwen3Config
    from pylon_b200.weights import write_random_model

    folders = {}
    for name, fields in TINY_CONFIGS.items():
        folder = tmp_path_factory.mktemp(name)
        write_random_model(Qwen3Config(**fields), TINY_SEEDS[name], folder, dtype="bfloat16")
        folders[name] = folder
    return folders
