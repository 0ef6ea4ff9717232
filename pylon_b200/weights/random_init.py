"""Random-weights mode: writes a model folder (``config.json``, ``model.safetensors``) from
a configuration and a seed.

Matrices and the embedding are N(0, 0.02); norm weights are 1 + N(0, 0.02).  Each tensor is
drawn from a generator seeded by (seed, tensor name), so a tensor's values do not depend on
which other tensors the model has or on the order they are written in.  raun6k/Pylon has no
such mode (its tests rely on torch's default initialisation under ``manual_seed``).
"""
from __future__ import annotations

import json
import zlib
from pathlib import Path
from typing import Any

import torch
from safetensors.torch import save_file

from pylon_b200.config.registry import ARCHITECTURES
from pylon_b200.models.decoder import DecoderModel

_STORE_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def random_tensor(name: str, shape: tuple[int, ...], role: str, seed: int) -> torch.Tensor:
    generator = torch.Generator(device="cpu")
    generator.manual_seed((int(seed) * 1_000_003 + zlib.crc32(name.encode())) % (2**63 - 1))
    values = torch.randn(shape, generator=generator, dtype=torch.float32) * 0.02
    return values + 1.0 if role == "vector" else values


def write_random_model(config: Any, seed: int, folder: str | Path, dtype: str = "bfloat16") -> Path:
    """Writes ``folder/config.json`` and ``folder/model.safetensors`` for ``config`` (a typed
    configuration of a registered architecture).  ``dtype`` is the storage type."""
    if dtype not in _STORE_DTYPES:
        raise ValueError(f"weights are stored as bfloat16 or float32, not {dtype}")
    architecture = ARCHITECTURES[config.architecture]
    model = DecoderModel(architecture.build_spec(config, 1))
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    tensors = {
        name: random_tensor(name, decl.shape, decl.role, seed).to(_STORE_DTYPES[dtype]).contiguous()
        for name, decl in model.tensor_decls().items()
    }
    save_file(tensors, str(folder / "model.safetensors"), metadata={"format": "pt"})
    data = config.to_dict()
    data["torch_dtype"] = dtype
    (folder / "config.json").write_text(json.dumps(data, indent=2) + "\n")
    return folder


def device_random_fetch(decls, seed: int, device: torch.device, dtype: torch.dtype):
    """A ``fetch(name)`` for :meth:`DecoderModel.load` that draws each tensor on the device:
    N(0, 0.02) matrices, 1 + N(0, 0.02) vectors, seeded by (seed, name).  The values differ
    from :func:`random_tensor`'s (another generator); the distributions are the same."""
    generator = torch.Generator(device=device)

    def fetch(name: str) -> torch.Tensor:
        decl = decls[name]
        generator.manual_seed((int(seed) * 1_000_003 + zlib.crc32(name.encode())) % (2**63 - 1))
        target = torch.float32 if decl.role == "vector" else dtype
        values = torch.empty(decl.shape, dtype=target, device=device)
        values.normal_(0.0, 0.02, generator=generator)
        return values + 1.0 if decl.role == "vector" else values

    return fetch
