"""Interfaces of the parts a layer is put together from, and their registries.

A part is built from a :class:`~pylon_b200.parts.spec.PartSpec` (its sizes and constants),
declares the checkpoint tensors it needs by name, receives them in ``load`` and then runs
on the device.  No part knows which model it is in: everything it needs at run time comes
through its constructor parameters, the :class:`StepView` of the current batch and the
:class:`LayerCache` the cache manager hands it.

Kinds of part and the interface each must have:

* **norm** (:class:`Norm`): ``apply(stream, rows=None) -> Tensor`` — fold the stream's
  pending delta into the residual and return the normalised activations.
* **position encoding** (:class:`PositionEncoding`): either ``rotary_table(device)``
  for encodings that are a per-position rotation of (query, key) pairs — the attention
  mixer then fuses them into its own kernel — or ``apply(q, k, step)`` for anything else.
* **mixer** (:class:`Mixer`): ``cache_need()`` says what it keeps between steps (paged keys
  and values, a fixed-size state, both or nothing); ``forward(h, step, cache) -> delta``.
* **feed-forward** (:class:`FeedForward`): ``forward(h, step) -> delta``.
* **block** (:class:`Block`): arranges a mixer, a feed-forward and its norms around the
  residual stream: ``forward(stream, step, cache)``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Mapping, Optional, Sequence

import torch

from pylon_b200.parts.spec import PartSpec


# ---------------------------------------------------------------------------------------
# tensors a part asks the loader for
# ---------------------------------------------------------------------------------------
@dataclass(frozen=True)
class TensorDecl:
    """A checkpoint tensor a part needs.  ``name`` is relative to the part's prefix.

    ``role`` decides how it is held on the device: ``matrix`` in the compute dtype
    (bfloat16 or float32), ``vector`` (norm weights and the like, used in 32-bit math)
    always in float32, ``table`` (integer tables) in int32.
    """

    name: str
    shape: tuple[int, ...]
    role: str = "matrix"


# ---------------------------------------------------------------------------------------
# what a mixer keeps between steps
# ---------------------------------------------------------------------------------------
@dataclass(frozen=True)
class KVNeed:
    """Paged rows per token: for each of ``n_kv_heads`` heads a key row of ``head_dim`` numbers and a
    value row of ``value_dim`` numbers (``None``: as wide as the key; ``0``: no value rows at all -
    a mixer that keeps one row per token, such as a compressed latent, asks for one head of
    that width and no values).

    ``window``: a query at position p reads keys at positions (p - window, p]; ``None``
    reads all of them.  Layers whose KVNeed is equal share a page pool (a cache group).
    """

    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    value_dim: Optional[int] = None

    @property
    def value_width(self) -> int:
        return self.head_dim if self.value_dim is None else self.value_dim


@dataclass(frozen=True)
class StateNeed:
    """A state of fixed size per request (``shape`` without the request dimension)."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass(frozen=True)
class CacheNeed:
    kv: Optional[KVNeed] = None
    state: Optional[StateNeed] = None


@dataclass
class LayerCache:
    """What the cache manager hands a mixer for one layer and one step.

    ``k_pages``: ``[num_pages, n_kv_heads, page_size, head_dim]`` of this layer; ``v_pages``
    likewise with the value rows' width, or ``None`` if the mixer asked for no value rows.  ``block_table``: int32 ``[rows, width]``, logical page of a row -> physical page
    (-1 where the row holds none, e.g. behind a window).  ``state``: ``[slots, *shape]``;
    a row's state is ``state[step.slots[row]]``.
    """

    k_pages: Optional[torch.Tensor] = None
    v_pages: Optional[torch.Tensor] = None
    block_table: Optional[torch.Tensor] = None
    page_size: int = 0
    state: Optional[torch.Tensor] = None


class StepView:
    """The batch of one step as the parts see it (all tensors on the device).

    token_ids   int32 [T]     the step's tokens, rows concatenated
    positions   int32 [T]     position of each token in its request
    token_row   int32 [T]     row (request of this step) of each token
    q_start     int32 [R+1]   first token of each row; q_start[R] == T
    kv_len      int32 [R]     tokens the request holds after this step
    slots       int32 [R]     state slot of each row's request
    logit_rows  int32 [L]     tokens whose logits are wanted
    num_tokens, num_rows, num_logits, max_q, max_kv: host integers (upper bounds when the
    step is replayed from a CUDA graph).
    row_tokens: the number of tokens each row brings, as host integers, for parts that plan
    their launches on the host; ``None`` when the step is replayed from a CUDA graph.
    rows_alike: the requests of the step hold about equally many tokens (within an eighth of the
    longest), so that work dealt out evenly by row is dealt out evenly; a hint, never needed for
    a right result.
    padded: the step was padded to the size of a captured CUDA graph.  It may then hold rows
    without tokens (``q_start[r + 1] == q_start[r]``, ``kv_len[r] == 0``, no pages) and, after
    the last row's tokens, padding tokens that belong to no row: ``token_row[t] == -1``, position
    0.  Whatever a part computes for a padding token is never read; it must keep nothing of it
    (no cache write, no state update).  Only models whose parts all say ``takes_padding`` get
    such steps.
    """

    token_ids: torch.Tensor
    positions: torch.Tensor
    token_row: torch.Tensor
    q_start: torch.Tensor
    kv_len: torch.Tensor
    slots: torch.Tensor
    logit_rows: torch.Tensor
    num_tokens: int
    num_rows: int
    num_logits: int
    max_q: int
    max_kv: int
    dtype: torch.dtype
    device: torch.device
    row_tokens: Optional[tuple] = None
    rows_alike: bool = False
    padded: bool = False


# ---------------------------------------------------------------------------------------
# base classes
# ---------------------------------------------------------------------------------------
class Part:
    """Common life cycle: construct from parameters, declare tensors, load, run."""

    def tensors(self) -> Sequence[TensorDecl]:
        return ()

    def load(self, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
        """``tensors``: name (as declared) -> tensor on the device, already in the dtype
        its role asks for."""

    def weight_bytes(self) -> int:
        """Bytes of device memory a step reads from this part's weights."""
        return 0


class Norm(Part):
    def apply(self, stream: "ResidualStream", rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    def rotary_table(self, device: torch.device) -> Optional[tuple[torch.Tensor, torch.Tensor, int]]:
        """(cos, sin, rotary_dim): float32 ``[positions, rotary_dim // 2]`` tables for
        encodings that rotate pairs ``(j, j + rotary_dim // 2)``; ``None`` otherwise."""
        return None

    def apply(self, q: torch.Tensor, k: torch.Tensor, step: StepView) -> None:
        """For encodings without such a table: change ``q [T, heads * d]`` and ``k [T, kv_heads * d]``
        (views with a row stride; already normalised if the mixer has q/k norms) in place, before
        ``k`` is written into the cache."""
        raise NotImplementedError


class Mixer(Part):
    # True if ``forward`` is right for a padded step (see :class:`StepView`): rows without tokens, tokens without a
    # row.  A mixer that indexes its cache or state by ``token_row`` has to look at this; so the default is False, and
    # a model with such a mixer is never padded.
    takes_padding = False

    def cache_need(self) -> CacheNeed:
        return CacheNeed()

    def forward(self, h: torch.Tensor, step: StepView, cache: LayerCache) -> torch.Tensor:
        """Returns the delta for the residual stream (see :class:`ResidualStream`)."""
        raise NotImplementedError


class FeedForward(Part):
    # A feed-forward works token by token, so padding tokens are usually no concern; one that looks across tokens (a
    # router that balances its load over the batch, say) sets this to False.
    takes_padding = True

    def forward(self, h: torch.Tensor, step: StepView) -> torch.Tensor:
        """Returns the delta for the residual stream (see :class:`ResidualStream`)."""
        raise NotImplementedError


class Block(Part):
    mixer: Mixer
    feed_forward: FeedForward

    @property
    def takes_padding(self) -> bool:
        return bool(self.mixer.takes_padding and self.feed_forward.takes_padding)

    def forward(self, stream: "ResidualStream", step: StepView, cache: LayerCache) -> None:
        raise NotImplementedError


class ResidualStream:
    """The residual sum in float32 ``[T, width]`` plus the delta not yet added to it.

    Parts hand their output to ``add``; the next norm folds it in (one fused kernel reads
    the delta once, updates the 32-bit sum and writes the normalised activations).  A delta
    is ``[T, width]`` in the activation dtype, or float32 partial sums ``[parts, T, width]``
    whose sum is the delta (what :func:`pylon_b200.kernels.ops.linear_for_residual` may return).
    """

    def __init__(self, residual: torch.Tensor) -> None:
        self.residual = residual
        self.pending: Optional[torch.Tensor] = None

    def add(self, delta: torch.Tensor) -> None:
        if self.pending is not None:
            self.flush()
        self.pending = delta

    def flush(self) -> None:
        if self.pending is not None:
            from pylon_b200.kernels import ops

            ops.residual_add(self.residual, self.pending)
            self.pending = None


# ---------------------------------------------------------------------------------------
# registries
# ---------------------------------------------------------------------------------------
class Registry:
    def __init__(self, what: str) -> None:
        self.what = what
        self._kinds: dict[str, Callable[..., Any]] = {}

    def register(self, kind: str) -> Callable[[Callable[..., Any]], Callable[..., Any]]:
        def decorate(factory: Callable[..., Any]) -> Callable[..., Any]:
            if kind in self._kinds and self._kinds[kind] is not factory:
                raise ValueError(f"{self.what} kind '{kind}' is registered already")
            self._kinds[kind] = factory
            return factory

        return decorate

    def unregister(self, kind: str) -> None:
        self._kinds.pop(kind, None)

    def build(self, spec: PartSpec, **extra: Any) -> Any:
        if spec.kind not in self._kinds:
            known = ", ".join(sorted(self._kinds)) or "none"
            raise KeyError(f"unknown {self.what} kind '{spec.kind}' (registered: {known})")
        return self._kinds[spec.kind](**dict(spec.params), **extra)

    def kinds(self) -> tuple[str, ...]:
        return tuple(sorted(self._kinds))


NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
BLOCKS = Registry("block")
