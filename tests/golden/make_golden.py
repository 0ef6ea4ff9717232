"""Makes tests/golden/*.npz: logits of raun6k/Pylon's own model code on two tiny random
Qwen3 models, computed on the CPU in float32.

Run once, by hand, where a checkout of raun6k/Pylon is at hand:

    python tests/golden/make_golden.py --reference <pylon checkout>/src

The reference is imported at run time (nothing of it is copied here).  Its loader insists
that ``lm_head.weight`` is absent and always ties the head to the embedding
(src/pylon/model/weights.py:36-39, src/pylon/model/model.py:32), so for the untied model
the head is assigned by hand after loading.  Its ``Decoder.verify_drafts``
(src/pylon/decode/runner.py:304-343) gives logits at every position of a packed batch.

Stored per model: the configuration, the prompts, logits at every position of every prompt
(whole prompts), and a checksum of every weight tensor, so that a change of the random
generator shows as a checksum mismatch, not as a numeric one.
"""
from __future__ import annotations

import argparse
import json
import sys
import tempfile
import zlib
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from pylon_b200.config import Qwen3Config  # noqa: E402
from pylon_b200.weights import write_random_model  # noqa: E402

TINY = {
    "tinyA": dict(
        config=dict(vocab_size=256, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                    head_dim=16, intermediate_size=128, max_position_embeddings=512, rope_theta=10_000.0,
                    rms_norm_eps=1e-6, tie_word_embeddings=True),
        seed=0, prompt_lengths=(5, 17, 33),
    ),
    "tinyB": dict(
        config=dict(vocab_size=320, hidden_size=96, num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=3,
                    head_dim=32, intermediate_size=224, max_position_embeddings=512, rope_theta=1_000_000.0,
                    rms_norm_eps=1e-5, tie_word_embeddings=False),
        seed=1, prompt_lengths=(1, 9, 24, 40),
    ),
}


def prompts_for(name: str) -> list[list[int]]:
    entry = TINY[name]
    rng = np.random.default_rng(entry["seed"])
    return [rng.integers(0, entry["config"]["vocab_size"], size=n).tolist() for n in entry["prompt_lengths"]]


def checksums(folder: Path) -> dict[str, int]:
    from safetensors import safe_open

    out = {}
    with safe_open(str(folder / "model.safetensors"), framework="pt") as handle:
        for name in sorted(handle.keys()):
            out[name] = zlib.crc32(handle.get_tensor(name).view(torch.uint8).numpy().tobytes())
    return out


def reference_logits(folder: Path, config: Qwen3Config, prompts: list[list[int]]) -> list[np.ndarray]:
    from safetensors.torch import load_file, save_file

    from pylon.decode.runner import Decoder
    from pylon.kv.cache import PagedKVCache
    from pylon.kv.pool import KVPagePool
    from pylon.model.config import Qwen3Config as ReferenceConfig
    from pylon.model.model import Qwen3Model
    from pylon.model.weights import Qwen3Weights

    ref_config = ReferenceConfig(
        vocab_size=config.vocab_size, context_length=config.max_position_embeddings, hidden_size=config.hidden_size,
        n_heads=config.num_attention_heads, n_layers=config.num_hidden_layers, hidden_dim=config.intermediate_size,
        head_dim=config.head_dim, n_kv_heads=config.num_key_value_heads, rope_theta=config.rope_theta,
        rms_norm_eps=config.rms_norm_eps, dtype=torch.float32,
    )
    tensors = load_file(str(folder / "model.safetensors"))
    head = tensors.pop("lm_head.weight", None)
    with tempfile.TemporaryDirectory() as scratch:
        save_file(tensors, str(Path(scratch) / "model.safetensors"))
        model = Qwen3Model(ref_config)
        Qwen3Weights(Path(scratch)).load_into(model)
    if head is not None:
        model.output.weight = torch.nn.Parameter(head.to(torch.float32))
    model.eval()
    decoder = Decoder(model)
    pool = KVPagePool(ref_config, 8, device=torch.device("cpu"), page_size=256)
    decoder.page_pool = pool
    outputs = []
    for prompt in prompts:
        cache = PagedKVCache(pool, len(prompt))
        rows = decoder.verify_drafts([cache], [prompt])
        outputs.append(rows[0].to(torch.float32).numpy().copy())
        cache.close()
    return outputs


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", required=True, help="the src folder of a raun6k/Pylon checkout")
    args = parser.parse_args()
    sys.path.insert(0, args.reference)
    here = Path(__file__).resolve().parent
    for name, entry in TINY.items():
        config = Qwen3Config(**entry["config"])
        prompts = prompts_for(name)
        with tempfile.TemporaryDirectory() as folder:
            folder = Path(folder)
            write_random_model(config, entry["seed"], folder, dtype="bfloat16")
            logits = reference_logits(folder, config, prompts)
            sums = checksums(folder)
        arrays = {f"logits_{i}": value for i, value in enumerate(logits)}
        arrays.update({f"prompt_{i}": np.asarray(p, dtype=np.int64) for i, p in enumerate(prompts)})
        np.savez_compressed(
            here / f"{name}.npz", meta=json.dumps({"config": entry["config"], "seed": entry["seed"], "checksums": sums}), **arrays
        )
        print(name, [a.shape for a in logits], "max |logit|", max(float(np.abs(a).max()) for a in logits))


if __name__ == "__main__":
    main()
