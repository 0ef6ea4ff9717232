"""Per-request sampling options.

``max_new_tokens``, ``temperature`` and ``top_p`` have raun6k/Pylon's names, ranges and
defaults (src/pylon/api/types.py:6-9).  ``seed``, ``stop_ids`` and ``ignore_eos`` are
additions: a seed makes a request's draws repeatable whatever it is batched with;
``ignore_eos`` lets benchmarks generate a fixed number of tokens.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class SamplingParams:
    max_new_tokens: int = 256
    temperature: float = 0.2
    top_p: float = 0.95
    seed: Optional[int] = None
    stop_ids: Optional[tuple[int, ...]] = None   # None: the model's eos ids
    ignore_eos: bool = False

    def __post_init__(self) -> None:
        if isinstance(self.max_new_tokens, bool) or not isinstance(self.max_new_tokens, int) or self.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be an integer of at least 1")
        if not 0 <= self.temperature <= 2:
            raise ValueError("temperature must be between 0 and 2")
        if not 0 < self.top_p <= 1:
            raise ValueError("top_p must be greater than 0 and at most 1")
        if self.stop_ids is not None:
            object.__setattr__(self, "stop_ids", tuple(int(t) for t in self.stop_ids))

    @property
    def greedy(self) -> bool:
        return self.temperature == 0
