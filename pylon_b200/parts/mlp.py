"""SwiGLU feed-forward: ``down(silu(gate(x)) * up(x))`` with gate and up as one product.

raun6k/Pylon's ``FeedForward`` (src/pylon/model/layers.py:13-27); the stacked ``[gate; up]``
layout is the one its loader builds (src/pylon/model/weights.py:65-67).
"""
from __future__ import annotations

from typing import Mapping, Optional, Sequence

import torch

from pylon_b200.kernels import ops
from pylon_b200.parts.base import FEED_FORWARDS, FeedForward, StepView, TensorDecl


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    def __init__(self, width: int, intermediate: int, names: Optional[Mapping[str, str]] = None) -> None:
        self.width, self.intermediate = int(width), int(intermediate)
        self.names = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight", **(names or {})}
        self.w_gate_up = self.w_down = None
        self.interleaved = False

    def tensors(self) -> Sequence[TensorDecl]:
        n = self.names
        return (
            TensorDecl(n["gate"], (self.intermediate, self.width)),
            TensorDecl(n["up"], (self.intermediate, self.width)),
            TensorDecl(n["down"], (self.width, self.intermediate)),
        )

    def load(self, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
        n = self.names
        # gate and up share one product.  In bfloat16 their rows alternate in groups of 8, so that
        # the product's kernel can apply silu(gate) * up itself; otherwise they lie in two halves.
        self.interleaved = dtype == torch.bfloat16 and self.intermediate % 8 == 0
        if self.interleaved:
            self.w_gate_up = ops.interleave_gate_up(tensors[n["gate"]], tensors[n["up"]])
        else:
            self.w_gate_up = torch.cat((tensors[n["gate"]], tensors[n["up"]]), dim=0).contiguous()
        self.w_down = tensors[n["down"]].contiguous()

    def weight_bytes(self) -> int:
        return (self.w_gate_up.numel() + self.w_down.numel()) * self.w_down.element_size()

    def forward(self, h: torch.Tensor, step: StepView) -> torch.Tensor:
        if self.interleaved:
            activation = ops.linear_swiglu(h, self.w_gate_up)
        else:
            activation = ops.swiglu(ops.linear(h, self.w_gate_up))
        return ops.linear_for_residual(activation, self.w_down)
