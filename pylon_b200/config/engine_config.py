"""Options of the engine (not of the model).

Where raun6k/Pylon has the option, the name, meaning and default are its own: it reads
them from ``PYLON_*`` environment variables (src/pylon/config.py:8-112), and so does
:meth:`EngineConfig.from_env`; the command line has the same names with dashes.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass, replace
from typing import Mapping, Optional

import torch

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def _env_bool(env: Mapping[str, str], name: str, default: bool) -> bool:
    value = env.get(name, str(default)).strip().lower()
    if value in {"1", "true"}:
        return True
    if value in {"0", "false"}:
        return False
    raise ValueError(f"{name} must be true, false, 1, or 0.")


@dataclass(frozen=True)
class EngineConfig:
    # raun6k/Pylon's options (src/pylon/config.py:8-27)
    prefill_chunk_size: int = 2048
    max_batch_size: int = 32
    max_queue_size: int = 32
    max_gpu_utilization: float = 0.90
    cuda_graphs: bool = False
    admit_skip: int = 4
    # this engine's own
    dtype: str = "bfloat16"            # "bfloat16": the serving kernels; "float32": everything in true 32-bit
    page_size: int = 256               # tokens per cache page (the reference's page, src/pylon/engine.py:26)
    max_cache_tokens: Optional[int] = None   # size of the page pool in tokens; None: from free memory
    max_context: Optional[int] = None  # longest request (prompt + new tokens); None: min(model limit, pool)
    seed: int = 0

    def __post_init__(self) -> None:
        if self.dtype not in _DTYPES:
            raise ValueError(f"dtype must be one of {sorted(_DTYPES)}, got {self.dtype!r}")
        if isinstance(self.prefill_chunk_size, bool) or not isinstance(self.prefill_chunk_size, int) or self.prefill_chunk_size < 1:
            raise ValueError("prefill_chunk_size must be a positive integer.")
        if self.max_batch_size < 1:
            raise ValueError("max_batch_size must be at least 1.")
        if self.max_queue_size < 1:
            raise ValueError("max_queue_size must be at least 1.")
        if not math.isfinite(self.max_gpu_utilization) or not 0 < self.max_gpu_utilization <= 1:
            raise ValueError("max_gpu_utilization must be greater than 0 and at most 1.")
        if isinstance(self.admit_skip, bool) or not isinstance(self.admit_skip, int) or self.admit_skip < 0:
            raise ValueError("admit_skip must be an integer of at least 0.")
        if self.page_size < 1:
            raise ValueError("page_size must be positive.")

    @property
    def torch_dtype(self) -> torch.dtype:
        return _DTYPES[self.dtype]

    @classmethod
    def from_env(cls, env: Optional[Mapping[str, str]] = None, **overrides) -> "EngineConfig":
        env = os.environ if env is None else env
        base = cls(
            prefill_chunk_size=int(env.get("PYLON_PREFILL_CHUNK_SIZE", "2048")),
            max_batch_size=int(env.get("PYLON_MAX_BATCH_SIZE", "32")),
            max_queue_size=int(env.get("PYLON_MAX_QUEUE_SIZE", "32")),
            max_gpu_utilization=float(env.get("PYLON_MAX_GPU_UTILIZATION", "0.90")),
            cuda_graphs=_env_bool(env, "PYLON_CUDA_GRAPHS", False),
            admit_skip=int(env.get("PYLON_ADMIT_SKIP", "4")),
        )
        return replace(base, **{key: value for key, value in overrides.items() if value is not None})
