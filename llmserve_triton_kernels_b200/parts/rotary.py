"""Rotary position encoding (half-rotation convention), unscaled.

Parity: src/llmserve/model/llama.py:31-54 — ``inv_freq[i] = 1 / theta**(2i/D)``, the angle of
position p is ``float32(p) * inv_freq[i]``, lanes ``j`` and ``j + D/2`` form a pair:
``x'[j] = x[j] cos - x[j+D/2] sin``, ``x'[j+D/2] = x[j+D/2] cos + x[j] sin``.  Angles, cosines
and sines are 32-bit.  They are tabulated once per model for positions ``0..max_positions-1``
with the same expression, so the kernels do no trigonometry and read ``[cos | sin]`` rows.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import PositionEncoding, register_part


_TABLES: dict = {}


class RotaryEmbedding(PositionEncoding):
    graph_safe = True
    rotary_layout = "half"  # lanes j and j + head_dim/2 form a pair, over the whole head

    def __init__(self, head_dim: int, theta: float, max_positions: int):
        if head_dim % 2:
            raise ValueError(f"rotary positions need an even head_dim, got {head_dim}")
        self.head_dim = int(head_dim)
        self.theta = float(theta)
        self.max_positions = int(max_positions)
        self.rotary_table: torch.Tensor | None = None  # [max_positions, head_dim]: cos | sin halves

    def bind(self, tensors, dtype, device) -> None:
        key = (self.head_dim, self.theta, self.max_positions, str(torch.device(device)))
        table = _TABLES.get(key)
        if table is None:  # layers with the same constants share one table
            exponent = torch.arange(0, self.head_dim, 2, dtype=torch.float32) / self.head_dim
            inv_freq = 1.0 / (self.theta**exponent)
            angles = torch.arange(self.max_positions, dtype=torch.float32)[:, None] * inv_freq
            table = _TABLES[key] = torch.cat((angles.cos(), angles.sin()), dim=-1).contiguous().to(device)
        self.rotary_table = table

    def apply(self, q, k, positions) -> None:
        ops.rope_inplace(q, positions, self.rotary_table)
        ops.rope_inplace(k, positions, self.rotary_table)


register_part("position", "rotary", RotaryEmbedding)
