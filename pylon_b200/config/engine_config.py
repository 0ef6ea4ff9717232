"""Options of the engine (not of the model).

Where raun6k/Pylon has the option, the name, meaning and default are its own: it reads
them from ``PYLON_*`` environment variables (src/pylon/config.py:8-112), and so does
:meth:`EngineConfig.from_env`; the command line has the same names with dashes.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass, fields, replace
from typing import Callable, Mapping, Optional

import torch

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}
_SWITCH_WORDS = {"1": True, "true": True, "0": False, "false": False}


def _whole_number(value: object) -> bool:
    return isinstance(value, int) and not isinstance(value, bool)


def _read_switch(text: str) -> bool:
    word = text.strip().lower()
    if word not in _SWITCH_WORDS:
        raise ValueError(f"a switch takes one of {sorted(_SWITCH_WORDS)}, not {text!r}")
    return _SWITCH_WORDS[word]


# option -> (environment variable, how its text is read); the defaults are the dataclass's own
_ENVIRONMENT: dict[str, tuple[str, Callable[[str], object]]] = {
    "prefill_chunk_size": ("PYLON_PREFILL_CHUNK_SIZE", int),
    "max_batch_size": ("PYLON_MAX_BATCH_SIZE", int),
    "max_queue_size": ("PYLON_MAX_QUEUE_SIZE", int),
    "max_gpu_utilization": ("PYLON_MAX_GPU_UTILIZATION", float),
    "cuda_graphs": ("PYLON_CUDA_GRAPHS", _read_switch),
    "admit_skip": ("PYLON_ADMIT_SKIP", int),
    "run_ahead": ("PYLON_B200_RUN_AHEAD", _read_switch),
}


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
    run_ahead: bool = True             # a tick queues its step before it waits for the tokens of the step before (see engine/scheduler.py)

    def __post_init__(self) -> None:
        if self.dtype not in _DTYPES:
            raise ValueError(f"dtype must be one of {sorted(_DTYPES)}, got {self.dtype!r}")
        lowest = {"prefill_chunk_size": 1, "max_batch_size": 1, "max_queue_size": 1, "page_size": 1, "admit_skip": 0}
        for name, least in lowest.items():
            value = getattr(self, name)
            if not _whole_number(value) or value < least:
                raise ValueError(f"{name} = {value!r}: a whole number, {least} or more, is needed")
        share = self.max_gpu_utilization
        if not isinstance(share, (int, float)) or isinstance(share, bool) or not math.isfinite(share) or not 0 < share <= 1:
            raise ValueError(f"max_gpu_utilization = {share!r}: a share of the device's memory, above 0 and up to 1, is needed")
        for name in ("max_cache_tokens", "max_context"):
            value = getattr(self, name)
            if value is not None and (not _whole_number(value) or value < 1):
                raise ValueError(f"{name} = {value!r}: a whole number of tokens, 1 or more, or None")

    @property
    def torch_dtype(self) -> torch.dtype:
        return _DTYPES[self.dtype]

    @classmethod
    def from_env(cls, env: Optional[Mapping[str, str]] = None, **overrides) -> "EngineConfig":
        """The options the environment gives (``env``: a mapping; default ``os.environ``), then ``overrides``
        that are not ``None``.  An option the environment does not name keeps its default."""
        env = os.environ if env is None else env
        known = {f.name for f in fields(cls)}
        found = {}
        for option, (variable, read) in _ENVIRONMENT.items():
            text = env.get(variable)
            if text is None:
                continue
            try:
                found[option] = read(text)
            except ValueError as error:
                raise ValueError(f"{variable}={text!r} cannot be read: {error}") from None
        for option, value in overrides.items():
            if option not in known:
                raise TypeError(f"EngineConfig has no option {option!r}")
            if value is not None:
                found[option] = value
        return replace(cls(), **found)
