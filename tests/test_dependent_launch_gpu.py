"""A step of several prompt portions and no decoded row, large enough for several waves of
blocks, with programmatic dependent launch on and off.

In such a step the decode attention has no row of its own.  A kernel in a chain of dependent
launches that ends without waiting for the kernel ahead of it lets the kernel after it start
reading before that one has finished writing; the tiny models finish in one wave and cannot
show it.  Both runs must give the plain implementation's logits, and the same logits as
each other."""
from __future__ import annotations

import os

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
import trace_tools

pytestmark = pytest.mark.gpu

CONFIG = dict(vocab_size=4_096, hidden_size=1_024, num_hidden_layers=2, num_attention_heads=16, num_key_value_heads=4, head_dim=128,
              intermediate_size=2_816, max_position_embeddings=1_024, rope_theta=1_000_000.0, rms_norm_eps=1e-6, tie_word_embeddings=False)
LENGTHS = (500, 433, 512, 390, 471, 505, 448, 497)


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    from pylon_b200.config import Qwen3Config
    from pylon_b200.weights import write_random_model

    folder = tmp_path_factory.mktemp("portions")
    write_random_model(Qwen3Config(**CONFIG), 11, folder)
    cfg, weights = plain.read_model(folder, torch.float64)
    weights = {name: tensor.cuda() for name, tensor in weights.items()}
    rng = np.random.default_rng(5)
    requests = {f"p{i}": rng.integers(0, CONFIG["vocab_size"], size=n).tolist() for i, n in enumerate(LENGTHS)}
    with torch.no_grad():
        expected = {rid: plain.forward(cfg, weights, tokens).cpu().numpy() for rid, tokens in requests.items()}
    return folder, requests, expected


def test_several_portions_in_one_step_with_and_without_dependent_launch(model, tmp_path):
    folder, requests, expected = model
    # the same step three times over (under new names), so that the kernels of one step follow those of the last closely
    steps = [{"step": index, "entries": [{"id": f"{rid}.{index}", "tokens": tokens, "want": list(range(len(tokens)))} for rid, tokens in requests.items()],
              "end": [f"{rid}.{index}" for rid in requests]} for index in range(3)]
    results = {}
    for mode in ("1", "0"):
        env = dict(os.environ, PYLON_B200_PDL=mode)
        results[mode] = trace_tools.run_program(folder, "bfloat16", steps, tmp_path / f"pdl{mode}", max_tokens=sum(-(-n // 64) * 64 for n in LENGTHS), env=env)
    for mode, got in results.items():
        for name, logits in got.items():
            rid = name.split(".")[0]
            error = logits.astype(np.float64) - expected[rid]
            rms = float(np.sqrt((error**2).mean()))
            assert rms < 0.01 and np.abs(error).max() < 0.08, (mode, name, rms, np.abs(error).max())
    first = results["0"]
    for mode, got in results.items():
        for name, logits in got.items():
            assert np.array_equal(logits, first[name.split(".")[0] + ".0"]), f"{name}, dependent launch {mode}: the logits depend on it or on the run"
