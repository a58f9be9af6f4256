"""A model as data: layers named by their parts, and the order in which they run."""

from __future__ import annotations

from dataclasses import dataclass
from types import MappingProxyType
from typing import Mapping

from ..parts.base import PartSpec


class LayerSpec:
    """One layer: the kind of block that arranges it, and the parts that block asks for, by role.

    Which roles there are is the block kind's business (``Block.roles``: role -> part category): the pre-norm block
    has ``mixer_norm, mixer, ff_norm, feed_forward``; a block with norms after its parts as well, or with one norm and
    two parallel parts, names other roles and is built from the same ``LayerSpec(block, role=spec, ...)``."""

    __slots__ = ("block", "parts")

    def __init__(self, block: PartSpec, parts: Mapping[str, PartSpec] | None = None, **roles: PartSpec):
        object.__setattr__(self, "block", block)
        object.__setattr__(self, "parts", MappingProxyType({**(parts or {}), **roles}))

    def __setattr__(self, name, value):
        raise AttributeError("a LayerSpec is not changed after it is made")

    def __getattr__(self, role: str) -> PartSpec:  # spec.mixer, spec.ff_norm, ...
        try:
            return self.parts[role]
        except KeyError:
            raise AttributeError(role) from None

    def replace(self, block: PartSpec | None = None, **roles: PartSpec) -> "LayerSpec":
        """A copy with another block or other parts in the named roles."""
        return LayerSpec(block or self.block, {**self.parts, **roles})

    def __eq__(self, other) -> bool:
        return isinstance(other, LayerSpec) and self.block == other.block and dict(self.parts) == dict(other.parts)

    def __hash__(self) -> int:
        return hash((self.block.kind, tuple(self.parts)))

    def __repr__(self) -> str:
        return f"LayerSpec({self.block!r}, {dict(self.parts)!r})"


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
    ignored: tuple[str, ...] = ()  # names a checkpoint may carry that the model does not read (e.g. a copy of a tied head)

    def __post_init__(self) -> None:
        for i, run in enumerate(self.schedule):
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"schedule entry {i} names layer {run.layer}, of {len(self.layers)}")
            if run.cache_of is not None:
                if not 0 <= run.cache_of < i:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {run.cache_of}, which is not earlier")
                if self.schedule[run.cache_of].cache_of is not None:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {run.cache_of}, which keeps none itself")
