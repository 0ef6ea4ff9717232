"""Block arrangements: how a mixer, a feed-forward and their norms sit on the residual stream.

``prenorm`` is raun6k/Pylon's ``TransformerBlock`` (src/pylon/model/layers.py:168-200):
``x += mixer(norm1(x)); x += ffn(norm2(x))``.  The adds are deferred to the next norm
(see :class:`~pylon_b200.parts.base.ResidualStream`).
"""
from __future__ import annotations

from typing import Mapping, Optional, Sequence

import torch

from pylon_b200.parts.base import (
    BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, LayerCache, ResidualStream, StepView, TensorDecl,
)
from pylon_b200.parts.spec import PartSpec


def _prefixed(prefix: str, decls: Sequence[TensorDecl]) -> list[TensorDecl]:
    return [TensorDecl(prefix + d.name, d.shape, d.role) for d in decls]


def _strip(prefix: str, tensors: Mapping[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    return {name[len(prefix):]: tensor for name, tensor in tensors.items() if name.startswith(prefix)}


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    """Sub-parts keep their tensors under the given sub-prefixes of the layer's prefix."""

    def __init__(
        self,
        mixer: PartSpec,
        feed_forward: PartSpec,
        mixer_norm: PartSpec,
        ffn_norm: PartSpec,
        mixer_prefix: str = "self_attn.",
        ffn_prefix: str = "mlp.",
        mixer_norm_prefix: str = "input_layernorm.",
        ffn_norm_prefix: str = "post_attention_layernorm.",
    ) -> None:
        self.mixer = MIXERS.build(mixer)
        self.feed_forward = FEED_FORWARDS.build(feed_forward)
        self.mixer_norm = NORMS.build(mixer_norm)
        self.ffn_norm = NORMS.build(ffn_norm)
        self._children = (
            (mixer_prefix, self.mixer), (ffn_prefix, self.feed_forward),
            (mixer_norm_prefix, self.mixer_norm), (ffn_norm_prefix, self.ffn_norm),
        )

    def tensors(self) -> Sequence[TensorDecl]:
        return [decl for prefix, part in self._children for decl in _prefixed(prefix, part.tensors())]

    def load(self, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
        for prefix, part in self._children:
            part.load(_strip(prefix, tensors), dtype, device)

    def weight_bytes(self) -> int:
        return sum(part.weight_bytes() for _, part in self._children)

    def forward(self, stream: ResidualStream, step: StepView, cache: LayerCache) -> None:
        stream.add(self.mixer.forward(self.mixer_norm.apply(stream), step, cache))
        stream.add(self.feed_forward.forward(self.ffn_norm.apply(stream), step))
