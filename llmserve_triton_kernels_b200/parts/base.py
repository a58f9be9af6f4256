"""The interfaces that layers are put together from, and the registry of part kinds.

A model is data: a list of layers, each naming its parts (a mixer, a feed-forward, two norms,
optionally a position encoding inside the mixer) by *kind* with their constants as plain
parameters, plus the order in which the layers run.  A part never sees a model configuration;
it gets its sizes and constants through its constructor, declares the tensors it owns by local
name, and is handed them once they are loaded.

Interfaces (what a new part must provide):

* every part: ``tensors() -> {local name: TensorSpec}`` and ``bind(tensors, dtype, device)``;
* ``Norm``: ``forward(x) -> y`` (and optionally the fused ``add_forward``);
* ``PositionEncoding``: ``apply(q, k, positions)`` in place on ``[N, heads, head_dim]`` views;
* ``Mixer``: ``cache_spec()`` saying what it keeps per request (pages of keys and values, a
  slot of fixed-size state, or nothing) and ``forward(x, ctx, cache) -> delta``;
* ``FeedForward``: ``forward(x, ctx) -> delta``;
* ``Block``: ``roles`` (which parts it is built from) and ``forward(resid, pending, ctx, cache) -> pending``
  arranging them.

The reference hard-wires these choices into classes that read one config object
(src/llmserve/model/llama.py:57-135); here they are parameters.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

import torch


@dataclass(frozen=True)
class TensorSpec:
    """One tensor a part owns: its shape and how a random model fills it."""

    shape: tuple[int, ...]
    init: str = "normal"  # "normal": N(0, std); "ones_plus_normal": 1 + N(0, std); "zeros"
    optional: bool = False  # absent from a checkpoint without error (e.g. a tied head)


@dataclass(frozen=True)
class PartSpec:
    """A part chosen by kind, with its constants and the prefix of its tensor names."""

    kind: str
    params: dict[str, Any] = field(default_factory=dict)
    prefix: str = ""


@dataclass(frozen=True)
class PagedKVSpec:
    """A mixer that keeps keys and values of ``kv_heads x head_dim`` for every token (``window``
    None) or for the last ``window`` tokens only."""

    kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class StateSpec:
    """A mixer that keeps one tensor of fixed shape per request, zeroed when the request starts."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Part:
    category = "part"
    # True if forward() launches the same device work for the same shapes whatever the step's
    # contents (no reads of device data on the host, no host loops over lengths): then a decode
    # step through this part can be captured in a CUDA graph.  A captured step's first run is an
    # ordinary pass and every later one a replay, so each step runs exactly once.
    graph_safe = False

    def tensors(self) -> dict[str, TensorSpec]:
        return {}

    def bind(self, tensors: dict[str, torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
        """Take ownership of the loaded tensors (keyed by local name), in the compute dtype."""


class Norm(Part):
    category = "norm"

    def forward(self, x: torch.Tensor, rows: torch.Tensor | None = None) -> torch.Tensor:
        """Normalise the rows of ``x`` (or only the rows listed in ``rows``) into the compute dtype."""
        raise NotImplementedError

    def add_forward(
        self, resid: torch.Tensor, delta: torch.Tensor | None, rows: torch.Tensor | None = None
    ) -> torch.Tensor:
        """``resid += delta`` in 32-bit, then normalise.  With ``rows`` only those rows are
        produced and ``resid`` is left as it was.  A norm may fuse the two; this default does not."""
        if delta is not None:
            if rows is None:
                resid.add_(delta.to(resid.dtype))
            else:
                return self.forward(resid[rows.long()] + delta[rows.long()].to(resid.dtype))
        return self.forward(resid, rows)


class PositionEncoding(Part):
    category = "position"
    # How a tabulated rotation pairs the lanes of a head, for mixers whose kernels can apply it while they store keys
    # and values: "half" = lanes (j, j + head_dim/2) over the whole head, with ``rotary_table [positions, head_dim]`` =
    # cos | sin halves.  None (or a layout a mixer does not know): the mixer calls ``apply``.
    rotary_layout: str | None = None

    def apply(self, q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor) -> None:
        """Encode absolute ``positions [N]`` into ``q [N, H, D]`` and ``k [N, KV, D]`` in place."""
        raise NotImplementedError


class Mixer(Part):
    category = "mixer"

    def cache_spec(self) -> PagedKVSpec | StateSpec | None:
        return None

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        """``x [N, hidden]`` (normalised) -> the mixer's contribution to the residual ``[N, hidden]``.
        ``ctx`` is the step's :class:`StepContext`; ``cache`` what the cache manager holds for this
        run of the layer (a ``PagedKVView``, a ``StateView`` or None)."""
        raise NotImplementedError


class FeedForward(Part):
    category = "feed_forward"

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    """The arrangement of norms, mixer and feed-forward around the residual stream.

    ``roles`` names the parts a block kind is built from and the category of each, in the order of its
    constructor's arguments: the model builds one part per role from the layer's ``LayerSpec`` and hands them over by
    these names.  A block kind with more norms, or with parts side by side, declares other roles."""

    category = "block"
    roles: dict[str, str] = {}

    def owned_parts(self) -> list[Part]:
        """The parts of this block, in the order of ``roles``."""
        return [getattr(self, role) for role in self.roles]

    def first_norm(self):
        """The norm that the residual stream meets first in this block (None: it meets none first), so that the
        block in front may fold it into its last product."""
        return getattr(self, "mixer_norm", None)

    def cache_spec(self):
        """What this block keeps per request: its mixer's ``cache_spec()``."""
        return self.mixer.cache_spec()

    def forward(self, resid: torch.Tensor, pending, ctx, cache, next_norm=None):
        """``resid [N, hidden]`` is the 32-bit residual stream, updated in place; ``pending`` a
        contribution not yet added to it.  Returns the new pending contribution.  ``next_norm`` is
        the norm that the stream meets after this block (None after the last); a block may use it
        to fuse that norm into its last product, and must expose its own first norm as
        ``mixer_norm`` and its mixer as ``mixer``."""
        raise NotImplementedError


_REGISTRY: dict[str, dict[str, Callable[..., Part]]] = {
    "norm": {},
    "position": {},
    "mixer": {},
    "feed_forward": {},
    "block": {},
}


def register_part(category: str, kind: str, factory: Callable[..., Part] | None = None):
    """Register ``factory(**params) -> Part`` under ``(category, kind)``; usable as a decorator."""
    if category not in _REGISTRY:
        raise KeyError(f"unknown part category {category!r}; known: {sorted(_REGISTRY)}")

    def _add(f):
        _REGISTRY[category][kind] = f
        return f

    return _add(factory) if factory is not None else _add


def part_factory(category: str, kind: str) -> Callable[..., Part]:
    kinds = _REGISTRY[category]
    if kind not in kinds:
        raise KeyError(f"no {category} of kind {kind!r} is registered; known: {sorted(kinds)}")
    return kinds[kind]


def build_part(category: str, spec: PartSpec, **more) -> Part:
    return part_factory(category, spec.kind)(**spec.params, **more)
