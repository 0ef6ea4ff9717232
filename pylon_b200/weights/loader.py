"""Reads checkpoint tensors by name from safetensors files of a model folder.

The folder holds ``model.safetensors``, or shards named by
``model.safetensors.index.json`` (discovery as raun6k/Pylon's
src/pylon/model/weights.py:41-49).  Tensors come back exactly as stored: bfloat16 stays
bfloat16, a tensor stored in 32 bits stays so, integer tables become int32; what dtype a
tensor has on the device is the business of the part that owns it.

Before anything is copied, the names and shapes in the files are compared with what the
model declares, and all differences are reported at once: missing tensors, unexpected
tensors and wrong shapes in one :class:`WeightError`.  (The reference stops at the first
wrong shape, ignores unknown names and insists that ``lm_head.weight`` is absent,
src/pylon/model/weights.py:24-39.)
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Iterable, Mapping

import torch
from safetensors import safe_open

from pylon_b200.parts.base import TensorDecl


class WeightError(ValueError):
    """The checkpoint does not hold what the model needs."""

    def __init__(self, folder, missing, unexpected, wrong_shape) -> None:
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong_shape = sorted(wrong_shape)
        lines = [f"checkpoint in {folder} does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(
                f"{name}: expected {tuple(expected)}, found {tuple(found)}" for name, expected, found in self.wrong_shape))
        super().__init__("\n".join(lines))


def shard_files(folder: Path) -> list[Path]:
    index = folder / "model.safetensors.index.json"
    if index.is_file():
        names = sorted(set(json.loads(index.read_text())["weight_map"].values()))
        return [folder / name for name in names]
    single = folder / "model.safetensors"
    if not single.is_file():
        raise FileNotFoundError(f"{folder} holds neither model.safetensors nor model.safetensors.index.json")
    return [single]


class Checkpoint:
    """Open safetensors files of one folder; tensors are read one at a time on request."""

    def __init__(self, folder: str | Path) -> None:
        self.folder = Path(folder)
        self._handles = [safe_open(str(path), framework="pt", device="cpu") for path in shard_files(self.folder)]
        self._where: dict[str, int] = {}
        for number, handle in enumerate(self._handles):
            for name in handle.keys():
                self._where[name] = number

    def names(self) -> Iterable[str]:
        return self._where.keys()

    def shape(self, name: str) -> tuple[int, ...]:
        return tuple(self._handles[self._where[name]].get_slice(name).get_shape())

    def verify(self, decls: Mapping[str, TensorDecl], ignored: Iterable[str] = ()) -> None:
        """Raises one :class:`WeightError` listing every difference from ``decls``."""
        ignored = set(ignored)
        present = set(self._where)
        missing = set(decls) - present
        unexpected = present - set(decls) - ignored
        wrong = [
            (name, decl.shape, self.shape(name))
            for name, decl in decls.items()
            if name in present and self.shape(name) != tuple(decl.shape)
        ]
        if missing or unexpected or wrong:
            raise WeightError(self.folder, missing, unexpected, wrong)

    def fetch(self, name: str) -> torch.Tensor:
        tensor = self._handles[self._where[name]].get_tensor(name)
        if tensor.dtype in (torch.int64, torch.int16, torch.int8, torch.uint8):
            tensor = tensor.to(torch.int32)
        return tensor
