"""A decoder put together from a :class:`~pylon_b200.parts.spec.ModelSpec`.

Embedding, the layers in their run order, final norm and vocabulary head.  The class knows
no architecture: which parts a layer has, their sizes and the order of the runs all come
from the spec.  The data flow is raun6k/Pylon's packed forward
(src/pylon/model/model.py:124-144): embed, blocks, then norm and head only at the rows
whose logits are wanted.  Two things architectures do around that flow are constants of the
spec: a factor on the embedding rows, and a factor and a soft cap on the logits.
"""
from __future__ import annotations

from typing import Callable, Mapping, Optional, Sequence

import torch

from pylon_b200.kernels import ops
from pylon_b200.parts.base import BLOCKS, NORMS, CacheNeed, LayerCache, ResidualStream, StepView, TensorDecl
from pylon_b200.parts.spec import ModelSpec

_ROLE_DTYPES = {"vector": torch.float32, "table": torch.int32}


class DecoderModel:
    def __init__(self, spec: ModelSpec) -> None:
        self.spec = spec
        self.blocks = [BLOCKS.build(layer.block) for layer in spec.layers]
        self.final_norm = NORMS.build(spec.final_norm)
        self.embedding: Optional[torch.Tensor] = None
        self.lm_head: Optional[torch.Tensor] = None
        self.dtype: Optional[torch.dtype] = None
        self.device: Optional[torch.device] = None

    # -- weights -------------------------------------------------------------------------
    def tensor_decls(self) -> dict[str, TensorDecl]:
        """Every checkpoint tensor the model needs, by full name."""
        spec = self.spec
        decls = {spec.embedding_name: TensorDecl(spec.embedding_name, (spec.vocab_size, spec.width))}
        if spec.lm_head_name is not None:
            decls[spec.lm_head_name] = TensorDecl(spec.lm_head_name, (spec.vocab_size, spec.width))
        for decl in self.final_norm.tensors():
            name = spec.final_norm_prefix + decl.name
            decls[name] = TensorDecl(name, decl.shape, decl.role)
        for layer, block in zip(spec.layers, self.blocks):
            for decl in block.tensors():
                name = layer.prefix + decl.name
                if name in decls:
                    raise ValueError(f"two parts declare the tensor '{name}'")
                decls[name] = TensorDecl(name, decl.shape, decl.role)
        return decls

    def load(self, fetch: Callable[[str], torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
        """``fetch(name)`` returns a checkpoint tensor as stored (host memory).  Tensors are
        moved part by part so that host and device never hold a second copy of the model."""
        self.dtype, self.device = dtype, torch.device(device)

        def place(decl: TensorDecl) -> torch.Tensor:
            target = _ROLE_DTYPES.get(decl.role, dtype)
            return fetch(decl.name).to(device=self.device, dtype=target)

        spec = self.spec
        decls = self.tensor_decls()
        self.embedding = place(decls[spec.embedding_name]).contiguous()
        self.lm_head = self.embedding if spec.lm_head_name is None else place(decls[spec.lm_head_name]).contiguous()
        self.final_norm.load(
            {decl.name: place(decls[spec.final_norm_prefix + decl.name]) for decl in self.final_norm.tensors()}, dtype, self.device
        )
        for layer, block in zip(spec.layers, self.blocks):
            block.load({decl.name: place(decls[layer.prefix + decl.name]) for decl in block.tensors()}, dtype, self.device)

    def weight_bytes(self) -> int:
        """Bytes of weights one step reads (each layer once per run; the head once)."""
        total = self.lm_head.numel() * self.lm_head.element_size() + self.final_norm.weight_bytes()
        for run in self.spec.order:
            total += self.blocks[run.layer].weight_bytes()
        return total

    def takes_padding(self) -> bool:
        """Whether every layer that runs is right for steps padded to the size of a captured graph."""
        return all(self.blocks[run.layer].takes_padding for run in self.spec.order)

    # -- cache ---------------------------------------------------------------------------
    def cache_needs(self) -> list[Optional[CacheNeed]]:
        """Per run of the order: what its mixer keeps between steps (``None`` where the run
        reads another run's cache)."""
        return [
            None if run.cache_of is not None else self.blocks[run.layer].mixer.cache_need()
            for run in self.spec.order
        ]

    # -- run -----------------------------------------------------------------------------
    def forward(self, step: StepView, caches: Sequence[LayerCache]) -> Optional[torch.Tensor]:
        """Runs the step's tokens; returns float32 logits ``[num_logits, vocab]`` at
        ``step.logit_rows`` (``None`` when no logits are wanted: the head is skipped).
        ``caches[i]`` belongs to run ``i`` of the order (a shared cache appears twice)."""
        residual = ops.embed_gather(step.token_ids, self.embedding, scale=self.spec.embedding_scale)
        stream = ResidualStream(residual)
        for position, run in enumerate(self.spec.order):
            self.blocks[run.layer].forward(stream, step, caches[position])
        if step.num_logits == 0:
            return None
        hidden = self.final_norm.apply(stream, rows=step.logit_rows)
        logits = ops.linear(hidden, self.lm_head, out_dtype=torch.float32)
        if self.spec.logit_scale != 1.0 or self.spec.logit_softcap is not None:
            ops.logit_transform(logits, self.spec.logit_scale, self.spec.logit_softcap)
        return logits
