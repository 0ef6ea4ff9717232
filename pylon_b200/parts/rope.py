"""Rotary position encoding.

Tables as raun6k/Pylon builds them (src/pylon/model/layers.py:43-51): float32
``inv_freq[j] = 1 / theta^(2j / d)``, ``angle[p, j] = p * inv_freq[j]`` formed in float32,
cos and sin of it; the rotation pairs element ``j`` with ``j + d/2`` (layers.py:73-78).
The tables stay float32 and the rotation is done in float32 inside the attention mixer's
fused kernel; only the first ``d/2`` columns are stored since both halves share angles.
"""
from __future__ import annotations

from typing import Optional

import torch

from pylon_b200.parts.base import POSITION_ENCODINGS, PositionEncoding


@POSITION_ENCODINGS.register("rope")
class RotaryEncoding(PositionEncoding):
    def __init__(self, head_dim: int, theta: float, max_positions: int, rotary_dim: Optional[int] = None) -> None:
        self.head_dim = int(head_dim)
        self.rotary_dim = int(rotary_dim if rotary_dim is not None else head_dim)
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary size {self.rotary_dim} must be even and at most the head size {self.head_dim}")
        self.theta = float(theta)
        self.max_positions = int(max_positions)
        self._tables: Optional[tuple[torch.Tensor, torch.Tensor]] = None

    def set_max_positions(self, positions: int) -> None:
        """The engine shortens the tables to the longest request it will hold."""
        if positions != self.max_positions:
            self.max_positions = int(positions)
            self._tables = None

    def rotary_table(self, device: torch.device):
        if self._tables is None or self._tables[0].device != device:
            exponent = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim
            inv_freq = 1.0 / (self.theta ** exponent)
            angles = torch.arange(self.max_positions, dtype=torch.float32).unsqueeze(1) * inv_freq.unsqueeze(0)
            self._tables = (torch.cos(angles).to(device).contiguous(), torch.sin(angles).to(device).contiguous())
        return self._tables[0], self._tables[1], self.rotary_dim
