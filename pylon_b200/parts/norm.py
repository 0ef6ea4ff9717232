"""RMSNorm over the residual stream.

``y = x / sqrt(mean(x^2) + eps) * weight`` in float32, as raun6k/Pylon's ``RMSNorm``
(src/pylon/model/layers.py:30-40).  The norm is where a pending delta joins the 32-bit
residual sum, so add and norm are one kernel.
"""
from __future__ import annotations

from typing import Mapping, Optional, Sequence

import torch

from pylon_b200.kernels import ops
from pylon_b200.parts.base import NORMS, Norm, ResidualStream, TensorDecl


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, width: int, eps: float, weight_name: str = "weight") -> None:
        self.width = int(width)
        self.eps = float(eps)
        self.weight_name = weight_name
        self.weight: Optional[torch.Tensor] = None
        self.dtype: Optional[torch.dtype] = None

    def tensors(self) -> Sequence[TensorDecl]:
        return (TensorDecl(self.weight_name, (self.width,), "vector"),)

    def load(self, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
        self.weight = tensors[self.weight_name].contiguous()
        self.dtype = dtype

    def weight_bytes(self) -> int:
        return self.width * 4

    def apply(self, stream: ResidualStream, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        delta, stream.pending = stream.pending, None
        # With a row selection the residual stays untouched and the delta is added on the fly.
        return ops.add_rmsnorm(stream.residual, delta, self.weight, self.eps, self.dtype, rows=rows)
