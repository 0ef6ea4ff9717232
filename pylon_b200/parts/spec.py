"""Architecture-neutral description of a model: what the part builders consume.

An architecture's configuration class turns its own ``config.json`` keys into a
:class:`ModelSpec`.  From here on nothing knows which architecture it is: a layer is a
block arrangement (a registered kind) of a mixer, a feed-forward and norms, each a
:class:`PartSpec` with its sizes and constants, chosen layer by layer.  The order in which
layers run is data as well: a list of :class:`RunSpec` that may name a layer twice (the
weights are shared, each run has a cache of its own) or let a run read the cache that an
earlier run owns.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from types import MappingProxyType
from typing import Any, Mapping, Optional, Union


@dataclass(frozen=True)
class PartSpec:
    """A registered part kind and the parameters its constructor takes."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def __post_init__(self) -> None:
        object.__setattr__(self, "params", MappingProxyType(dict(self.params)))

    def __hash__(self) -> int:
        return hash((self.kind, repr(sorted(self.params.items(), key=lambda item: item[0]))))


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement of parts and the checkpoint prefix of its tensors."""

    prefix: str        # e.g. "model.layers.3."
    block: PartSpec    # arrangement kind; its parameters name the mixer, feed-forward, norms


@dataclass(frozen=True)
class RunSpec:
    """One entry of the run order: which layer runs, and whose cache its mixer is handed.

    ``cache_of`` is the index of an earlier entry of the order that owns a cache; ``None``
    means this run owns its own (sized by what its mixer says it needs).
    """

    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    width: int                        # residual stream width
    vocab_size: int
    max_positions: int
    embedding_name: str               # checkpoint name of the [vocab, width] table
    lm_head_name: Optional[str]       # None: the head shares the embedding table
    final_norm: PartSpec
    final_norm_prefix: str
    layers: tuple[LayerSpec, ...]
    order: tuple[Union[RunSpec, int], ...]
    eos_token_ids: tuple[int, ...] = ()
    ignored_tensors: tuple[str, ...] = ()   # checkpoint names that may be present and are not used
    embedding_scale: float = 1.0            # the embedding rows are multiplied by it as they enter the residual stream
    logit_scale: float = 1.0                # the logits are multiplied by it,
    logit_softcap: Optional[float] = None   # then, with a cap c, squashed to c * tanh(logit / c)

    def __post_init__(self) -> None:
        runs = tuple(run if isinstance(run, RunSpec) else RunSpec(int(run)) for run in self.order)
        object.__setattr__(self, "order", runs)
        object.__setattr__(self, "layers", tuple(self.layers))
        if not runs:
            raise ValueError("a model must run at least one layer")
        for position, run in enumerate(runs):
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"run {position} names layer {run.layer}, but there are {len(self.layers)} layers")
            if run.cache_of is not None:
                if not 0 <= run.cache_of < position:
                    raise ValueError(f"run {position} reads the cache of run {run.cache_of}, which is not an earlier run")
                if runs[run.cache_of].cache_of is not None:
                    raise ValueError(f"run {position} reads the cache of run {run.cache_of}, which owns none")
