"""RMS normalisation with the residual sum fused in.

Parity: src/llmserve/model/llama.py:18-28 — mean of squares, ``+ eps`` and rsqrt in 32-bit,
then the weight multiply.  Here the residual stream itself is 32-bit and the result is rounded
once, after the weight multiply.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import Norm, TensorSpec, register_part


class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, size: int, eps: float):
        self.size = int(size)
        self.eps = float(eps)
        self.weight: torch.Tensor | None = None
        self.out_dtype: torch.dtype | None = None

    def tensors(self) -> dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.size,), init="ones_plus_normal")}

    def bind(self, tensors, dtype, device) -> None:
        self.weight = tensors["weight"].to(device=device, dtype=torch.float32).contiguous()
        self.out_dtype = dtype

    def fused_params(self):
        """``(weight, eps)``: what a product needs to fold this norm into its ends."""
        return self.weight, self.eps

    def forward(self, x, rows=None):
        return ops.rmsnorm(x, self.weight, self.eps, delta=None, rows=rows, out_dtype=self.out_dtype)

    def add_forward(self, resid, delta, rows=None):
        return ops.rmsnorm(resid, self.weight, self.eps, delta=delta, rows=rows, out_dtype=self.out_dtype)


register_part("norm", "rms_norm", RMSNorm)
