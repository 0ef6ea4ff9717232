"""The engine at the widths, head counts and vocabulary of Qwen3-4B, Qwen3-8B and Qwen3-14B (a group of
five query heads per KV head), with two layers so that the test stays short: float32 and
bfloat16 logits under several cuttings against the plain implementation run in float64 on the
GPU.  These sizes reach kernels the tiny models never do: head size 128, the tensor-core
products of long portions, the weight-streaming products of decode, a 151,936-wide head."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
import trace_tools

pytestmark = pytest.mark.gpu

SHAPES = {
    "4B": dict(vocab_size=151_936, hidden_size=2_560, num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
               intermediate_size=9_728, max_position_embeddings=4_096, rope_theta=5_000_000.0, rms_norm_eps=1e-6, tie_word_embeddings=True),
    "8B": dict(vocab_size=151_936, hidden_size=4_096, num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
               intermediate_size=12_288, max_position_embeddings=4_096, rope_theta=1_000_000.0, rms_norm_eps=1e-6, tie_word_embeddings=False),
    "14B": dict(vocab_size=151_936, hidden_size=5_120, num_hidden_layers=2, num_attention_heads=40, num_key_value_heads=8, head_dim=128,
                intermediate_size=17_408, max_position_embeddings=4_096, rope_theta=1_000_000.0, rms_norm_eps=1e-6, tie_word_embeddings=False),
}


@pytest.fixture(scope="module", params=list(SHAPES))
def big_model(request, tmp_path_factory):
    from pylon_b200.config import Qwen3Config
    from pylon_b200.weights import write_random_model

    folder = tmp_path_factory.mktemp(f"shape{request.param}")
    write_random_model(Qwen3Config(**SHAPES[request.param]), 3, folder)
    cfg, weights = plain.read_model(folder, torch.float64)
    weights = {name: tensor.cuda() for name, tensor in weights.items()}
    rng = np.random.default_rng(21)
    requests = {"long": rng.integers(0, 151_936, size=300).tolist(), "short": rng.integers(0, 151_936, size=37).tolist()}
    with torch.no_grad():
        expected = {rid: plain.forward(cfg, weights, tokens).cpu().numpy() for rid, tokens in requests.items()}
    del weights
    torch.cuda.empty_cache()
    return folder, requests, expected


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_big_shapes_under_cuttings(big_model, dtype):
    from pylon_b200.config import EngineConfig
    from pylon_b200.engine import Engine

    folder, requests, expected = big_model
    cuttings = {"whole": trace_tools.whole(requests), "tail": trace_tools.tail_one_by_one(requests, tail=12), "mixed": trace_tools.mixed(requests, seed=2, decode_tail=6)}
    engine = Engine(folder, EngineConfig(dtype=dtype, page_size=64, max_cache_tokens=1024, max_context=512, max_batch_size=4, cuda_graphs=dtype == "bfloat16"))
    # Logits are of order 1.  float32: sums of up to 17,408 products accumulate about sqrt(K) * 6e-8 relative error per
    # product and there are a dozen in a row, so a few 1e-5 is float32 rounding (a TF32 product would be off by 1e-3).
    # bfloat16: every activation is rounded to 8 bits of mantissa (0.2 to 0.4 %), which leaves logit errors with a
    # standard deviation near 0.01; a request has up to 45 million logits, whose largest error sits near six standard
    # deviations, so the check is on the root-mean-square error (0.02) and on the largest one (0.12), not on 0.05 each.
    for name, steps in cuttings.items():
        got = trace_tools.run_in_process(engine, steps)
        for rid in requests:
            if dtype == "float32":
                np.testing.assert_allclose(got[rid], expected[rid], err_msg=f"{name} {rid}", rtol=1e-4, atol=1e-4)
                continue
            error = got[rid].astype(np.float64) - expected[rid]
            assert np.sqrt((error**2).mean()) < 0.02 and np.abs(error).max() < 0.12, (name, rid, np.sqrt((error**2).mean()), np.abs(error).max())
            agree = (got[rid].argmax(-1) == expected[rid].argmax(-1)).mean()   # and the ranking survives at most positions
            assert agree > 0.8, (name, rid, agree)
    from pylon_b200.kernels import ops

    assert int(ops.tcgen05_error_word(torch.device("cuda")).item()) == 0
