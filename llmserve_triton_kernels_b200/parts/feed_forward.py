"""Dense gated feed-forward: ``down(act(gate(x)) * up(x))`` without biases.

Parity: src/llmserve/model/llama.py:112-120, where the activation is SiLU
(``z * sigmoid(z)``); the gate and up matrices are stacked at load so that one matrix product
feeds the activation kernel.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, TensorSpec, register_part

_ACTIVATIONS = ("silu",)


class GatedMLP(FeedForward):
    graph_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "silu", bias: bool = False):
        if activation not in _ACTIVATIONS:
            raise ValueError(f"activation {activation!r} is not built; known: {_ACTIVATIONS}")
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.activation = activation
        self.bias = bool(bias)  # ``*_proj.bias`` vectors (none in Llama): products and bias sums as kernels of their own
        self.b_gate_up: torch.Tensor | None = None
        self.b_down: torch.Tensor | None = None
        self.w_gate_up: torch.Tensor | None = None  # [2 I, hidden]: gate rows, then up rows
        self.w_down: torch.Tensor | None = None  # [hidden, I]

    def tensors(self) -> dict[str, TensorSpec]:
        i, h = self.intermediate_size, self.hidden_size
        specs = {
            "gate_proj.weight": TensorSpec((i, h)),
            "up_proj.weight": TensorSpec((i, h)),
            "down_proj.weight": TensorSpec((h, i)),
        }
        if self.bias:
            specs.update({"gate_proj.bias": TensorSpec((i,)), "up_proj.bias": TensorSpec((i,)), "down_proj.bias": TensorSpec((h,))})
        return specs

    def bind(self, tensors, dtype, device) -> None:
        fused = torch.cat([tensors["gate_proj.weight"].to(dtype), tensors["up_proj.weight"].to(dtype)], dim=0)
        self.w_gate_up = fused.to(device).contiguous()
        self.w_down = tensors["down_proj.weight"].to(device=device, dtype=dtype).contiguous()
        if self.bias:
            self.b_gate_up = torch.cat([tensors["gate_proj.bias"].to(dtype), tensors["up_proj.bias"].to(dtype)]).to(device).contiguous()
            self.b_down = tensors["down_proj.bias"].to(device=device, dtype=dtype).contiguous()

    accepts_sink = True

    def forward(self, x, ctx, sink=None):
        if self.bias:
            act = ops.swiglu(ops.add_bias(ops.linear(x, self.w_gate_up), self.b_gate_up))
            return ops.add_bias(ops.linear(act, self.w_down, out_dtype=torch.float32), self.b_down.float())
        act = ops.linear_swiglu(x, self.w_gate_up)
        if sink is not None:
            handed_on = sink.linear(act, self.w_down)
            if handed_on is not None:
                return handed_on
        # the contribution to the 32-bit residual stream leaves the product in 32-bit: it is the sum's largest addend
        return ops.linear(act, self.w_down, out_dtype=torch.float32)


register_part("feed_forward", "gated_mlp", GatedMLP)
