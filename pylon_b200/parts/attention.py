"""Grouped-query attention over the paged cache.

One fused QKV product (rows ``[q; k; v]``), optional per-head RMSNorm of q and k, the
position encoding, the write of k and v into the layer's pages, causal (optionally
windowed) attention over the pages, and the output product.  Order of operations as in
raun6k/Pylon's ``GroupedQueryAttention`` (src/pylon/model/layers.py:81-138) with its cache
write before attention (src/pylon/kv/cache.py:457-476).
"""
from __future__ import annotations

import math
from typing import Mapping, Optional, Sequence

import torch

from pylon_b200.kernels import ops
from pylon_b200.parts.base import (
    MIXERS, POSITION_ENCODINGS, CacheNeed, KVNeed, LayerCache, Mixer, StepView, TensorDecl,
)
from pylon_b200.parts.spec import PartSpec


@MIXERS.register("gqa_attention")
class GroupedQueryAttention(Mixer):
    takes_padding = True   # the kernels skip tokens without a row and rows without tokens

    def __init__(
        self,
        width: int,
        n_heads: int,
        n_kv_heads: int,
        head_dim: int,
        position: Optional[PartSpec] = None,
        qk_norm_eps: Optional[float] = None,
        window: Optional[int] = None,
        scale: Optional[float] = None,
        names: Optional[Mapping[str, str]] = None,
    ) -> None:
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} query heads cannot be grouped over {n_kv_heads} KV heads")
        self.width, self.n_heads, self.n_kv_heads, self.head_dim = int(width), int(n_heads), int(n_kv_heads), int(head_dim)
        self.q_size, self.kv_size = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        self.qk_norm_eps = None if qk_norm_eps is None else float(qk_norm_eps)
        self.window = None if window is None else int(window)
        self.scale = 1.0 / math.sqrt(self.head_dim) if scale is None else float(scale)
        self.position = POSITION_ENCODINGS.build(position) if position is not None else None
        self.names = {
            "q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
            "q_norm": "q_norm.weight", "k_norm": "k_norm.weight", **(names or {}),
        }
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = None

    # -- weights -------------------------------------------------------------------------
    def tensors(self) -> Sequence[TensorDecl]:
        n = self.names
        decls = [
            TensorDecl(n["q"], (self.q_size, self.width)),
            TensorDecl(n["k"], (self.kv_size, self.width)),
            TensorDecl(n["v"], (self.kv_size, self.width)),
            TensorDecl(n["o"], (self.width, self.q_size)),
        ]
        if self.qk_norm_eps is not None:
            decls += [TensorDecl(n["q_norm"], (self.head_dim,), "vector"), TensorDecl(n["k_norm"], (self.head_dim,), "vector")]
        return decls

    def load(self, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
        n = self.names
        # q, k and v share one product: their matrices are stacked by rows at load.
        self.w_qkv = torch.cat((tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]), dim=0).contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        if self.qk_norm_eps is not None:
            self.q_norm, self.k_norm = tensors[n["q_norm"]].contiguous(), tensors[n["k_norm"]].contiguous()

    def weight_bytes(self) -> int:
        return (self.w_qkv.numel() + self.w_o.numel()) * self.w_qkv.element_size() + (0 if self.q_norm is None else 8 * self.head_dim)

    # -- cache ---------------------------------------------------------------------------
    def cache_need(self) -> CacheNeed:
        return CacheNeed(kv=KVNeed(self.n_kv_heads, self.head_dim, self.window))

    # -- run -----------------------------------------------------------------------------
    def forward(self, h: torch.Tensor, step: StepView, cache: LayerCache) -> torch.Tensor:
        table = self.position.rotary_table(h.device) if self.position is not None else None
        cos, sin, rotary_dim = table if table is not None else (None, None, 0)
        q_norm, k_norm = self.q_norm, self.k_norm
        if self.position is not None and table is None:
            # An encoding that is not a rotation by a table runs as a step of its own, on normalised q and k and
            # before k goes into the cache; the fused kernel below is left with the cache write.
            qkv = ops.linear(h, self.w_qkv)
            if q_norm is not None:
                ops.qk_norm(qkv, q_norm, k_norm, self.qk_norm_eps, self.n_heads, self.n_kv_heads, self.head_dim)
                q_norm = k_norm = None
            self.position.apply(qkv[:, : self.q_size], qkv[:, self.q_size : self.q_size + self.kv_size], step)
        elif cos is not None and ops.qkv_rotation_fuses(h, self.w_qkv, self.head_dim, rotary_dim, cache.k_pages):
            qkv = None   # a long prompt portion: norms, rotation and cache write in the product's epilogue
        else:
            qkv = ops.linear_for_rotation(h, self.w_qkv, self.head_dim, rotary_dim)   # may be partial sums: the next kernel adds them
        if qkv is None:
            q = ops.linear_qkv_rotated(
                h, self.w_qkv, q_norm, k_norm, self.qk_norm_eps or 0.0, cos, sin, step.positions, step.token_row,
                cache.block_table, cache.page_size, cache.k_pages, cache.v_pages, self.n_heads, self.n_kv_heads, self.head_dim,
            )
        else:
            q = ops.qk_norm_rope_kv_write(
                qkv, q_norm, k_norm, self.qk_norm_eps or 0.0, cos, sin, rotary_dim, step.positions, step.token_row,
                cache.block_table, cache.page_size, cache.k_pages, cache.v_pages, self.n_heads, self.n_kv_heads, self.head_dim,
            )
        context = ops.paged_attention(
            q, cache.k_pages, cache.v_pages, step.positions, step.token_row, step.q_start, step.kv_len, cache.block_table,
            self.n_heads, step.max_q, step.max_kv, window=self.window, scale=self.scale, row_tokens=step.row_tokens,
            rows_alike=step.rows_alike,
        )
        return ops.linear_for_residual(context, self.w_o)
