"""A model as data: layers named by their parts, and the order in which they run."""

from __future__ import annotations

from dataclasses import dataclass

from ..parts.base import PartSpec


@dataclass(frozen=True)
class LayerSpec:
    """One layer's parts.  ``block`` arranges the other four around the residual stream."""

    block: PartSpec
    mixer_norm: PartSpec
    mixer: PartSpec
    ff_norm: PartSpec
    feed_forward: PartSpec


@dataclass(frozen=True)
class LayerRun:
    """One entry of the execution order.

    ``layer`` indexes ``ModelPlan.layers`` and may appear in several entries (the same weights
    run twice; each entry then keeps a cache of its own).  ``cache_of`` names an earlier entry
    of the order whose cache this entry reads instead of keeping one (shared keys and values).
    """

    layer: int
    cache_of: int | None = None


@dataclass(frozen=True)
class ModelPlan:
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: str  # tensor name of the token table [vocab, hidden]
    layers: tuple[LayerSpec, ...]
    schedule: tuple[LayerRun, ...]
    final_norm: PartSpec
    head: str | None  # tensor name of the output matrix [vocab, hidden]; None: the token table

    def __post_init__(self) -> None:
        for i, run in enumerate(self.schedule):
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"schedule entry {i} names layer {run.layer}, of {len(self.layers)}")
            if run.cache_of is not None:
                if not 0 <= run.cache_of < i:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {run.cache_of}, which is not earlier")
                if self.schedule[run.cache_of].cache_of is not None:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {run.cache_of}, which keeps none itself")
