"""One registry from an architecture's name (``config.json`` ``architectures[0]``) to its
typed configuration class and the function that describes its model.

raun6k/Pylon serves one hard-gated checkpoint (src/pylon/model/config.py:7,35-49) and has
no registry; here the name chooses, and an unknown name is an error that lists the known.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Mapping, Optional

from pylon_b200.config.model_config import ConfigError, Qwen3Config
from pylon_b200.parts.spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Any                                   # has from_dict(mapping) and to_dict()
    build_spec: Callable[[Any, Optional[int]], ModelSpec]  # (config, max_positions) -> ModelSpec


ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class: Any, build_spec: Callable[[Any, Optional[int]], ModelSpec]) -> None:
    ARCHITECTURES[name] = Architecture(name, config_class, build_spec)


def architecture_of(data: Mapping[str, Any]) -> Architecture:
    names = data.get("architectures")
    if not isinstance(names, (list, tuple)) or len(names) != 1 or not isinstance(names[0], str):
        raise ConfigError(f"config.json 'architectures' must name exactly one architecture, got {names!r}")
    if names[0] not in ARCHITECTURES:
        raise ConfigError(f"unknown architecture '{names[0]}' (known: {', '.join(sorted(ARCHITECTURES))})")
    return ARCHITECTURES[names[0]]


def read_config(model_dir: str | Path) -> tuple[Architecture, Any]:
    """Reads ``model_dir/config.json``; returns the architecture entry and its typed config."""
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path} does not exist")
    try:
        data = json.loads(path.read_text())
    except json.JSONDecodeError as error:
        raise ConfigError(f"{path} is not valid JSON: {error}") from error
    if not isinstance(data, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    architecture = architecture_of(data)
    return architecture, architecture.config_class.from_dict(data)


def _register_builtin() -> None:
    from pylon_b200.models.qwen3 import qwen3_spec

    register_architecture(Qwen3Config.architecture, Qwen3Config, qwen3_spec)


_register_builtin()
