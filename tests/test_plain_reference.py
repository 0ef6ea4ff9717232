"""The plain implementation against raun6k/Pylon's own model code (stored outputs), and
against itself (parts alone)."""
from __future__ import annotations

import json
import zlib
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from conftest import TINY_CONFIGS, TINY_SEEDS

GOLDEN = Path(__file__).resolve().parent / "golden"
# the prompts the stored outputs were made with: the requests of the two tiny benchmark configurations
GOLDEN_PROMPT_LENGTHS = {"tinyA": (5, 17, 33), "tinyB": (1, 9, 24, 40)}


@pytest.mark.parametrize("name", ["tinyA", "tinyB"])
def test_plain_matches_reference_outputs(name, tiny_folders):
    stored = np.load(GOLDEN / f"{name}.npz")
    meta = json.loads(str(stored["meta"]))
    assert meta["config"] == TINY_CONFIGS[name] and meta["seed"] == TINY_SEEDS[name]
    # the weights the goldens were made with are the weights the random mode writes today
    from safetensors import safe_open

    with safe_open(str(tiny_folders[name] / "model.safetensors"), framework="pt") as handle:
        assert sorted(handle.keys()) == sorted(meta["checksums"])
        for tensor_name, checksum in meta["checksums"].items():
            data = handle.get_tensor(tensor_name).view(torch.uint8).numpy().tobytes()
            assert zlib.crc32(data) == checksum, tensor_name
    cfg, weights = plain.read_model(tiny_folders[name])
    prompt_lengths = GOLDEN_PROMPT_LENGTHS[name]
    assert sorted(key for key in stored.files if key.startswith("prompt_")) == [f"prompt_{index}" for index in range(len(prompt_lengths))]
    for index, length in enumerate(prompt_lengths):
        prompt = stored[f"prompt_{index}"].tolist()
        assert len(prompt) == length
        logits = plain.as_numpy(plain.forward(cfg, weights, prompt))
        assert stored[f"logits_{index}"].shape == (length, cfg["vocab_size"])
        np.testing.assert_allclose(logits, stored[f"logits_{index}"], rtol=1e-4, atol=2e-6)


def test_rms_norm_is_scale_invariant_up_to_eps():
    x = torch.randn(4, 48, dtype=torch.float64)
    w = torch.rand(48, dtype=torch.float64) + 0.5
    a = plain.rms_norm(x, w, 0.0)
    b = plain.rms_norm(3.0 * x, w, 0.0)
    torch.testing.assert_close(a, b)
    assert torch.allclose((a / w).pow(2).mean(-1), torch.ones(4, dtype=torch.float64))


def test_rope_is_a_rotation_and_relative():
    torch.manual_seed(0)
    d = 32
    q = torch.randn(1, 6, d, dtype=torch.float64)
    k = torch.randn(1, 6, d, dtype=torch.float64)
    cos, sin = plain.rope_tables(d, 10_000.0, torch.arange(6), torch.float64)
    rq, rk = plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin)
    torch.testing.assert_close(rq.norm(dim=-1), q.norm(dim=-1))
    # the score of (query at p, key at p - 2) depends on the distance only
    cos2, sin2 = plain.rope_tables(d, 10_000.0, torch.arange(3, 9), torch.float64)
    sq, sk = plain.apply_rope(q, cos2, sin2), plain.apply_rope(k, cos2, sin2)
    torch.testing.assert_close((rq[0, 4] * rk[0, 2]).sum(), (sq[0, 4] * sk[0, 2]).sum(), atol=1e-5, rtol=1e-5)


def test_attention_mask_and_groups():
    torch.manual_seed(1)
    q = torch.randn(4, 5, 8, dtype=torch.float64)
    k = torch.randn(2, 5, 8, dtype=torch.float64)
    v = torch.randn(2, 5, 8, dtype=torch.float64)
    out = plain.causal_attention(q, k, v)
    # first token sees only itself: its output is v[0] of its KV head
    torch.testing.assert_close(out[3, 0], v[1, 0])
    torch.testing.assert_close(out[0, 0], v[0, 0])
    # a window of one sees only itself everywhere
    out1 = plain.causal_attention(q, k, v, window=1)
    torch.testing.assert_close(out1[2], v[1])
    # changing a later key does not change earlier outputs
    k2 = k.clone()
    k2[:, 4] += 1.0
    torch.testing.assert_close(plain.causal_attention(q, k2, v)[:, :4], out[:, :4])


def test_sampling_distribution_matches_reference_definition():
    torch.manual_seed(2)
    logits = torch.randn(50)
    probs = plain.sampling_distribution(logits, 0.8, 0.9)
    assert abs(float(probs.sum()) - 1.0) < 1e-12
    full = torch.softmax(logits.double() / 0.8, -1)
    order = torch.argsort(full, descending=True)
    mass_before = 0.0
    for rank, index in enumerate(order.tolist()):
        kept = rank == 0 or mass_before <= 0.9
        assert (probs[index] > 0) == kept
        mass_before += float(full[index])
    assert plain.greedy(torch.tensor([0.0, 2.0, 2.0, 1.0])) == 1
