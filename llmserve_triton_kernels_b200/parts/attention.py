"""Grouped-query attention over a paged cache of keys and values.

Parity: src/llmserve/model/llama.py:57-88 (projections without bias, rotary encoding of q and k
before the cache write, head-major concatenation into the output projection) and
src/llmserve/kvcache/paged.py:81-110 (key j is visible to the query at position p iff j <= p;
consecutive query heads share a key/value head; softmax scale 1/sqrt(head_dim), which arrives
here as the parameter ``scale``).  ``window`` (None in Llama) limits a query to the last
``window`` keys, itself included.  With ``own_kv=False`` the layer has no key and value
projections and reads the cache that an earlier layer of the order wrote.  ``qkv_bias`` and
``out_bias`` (both off in Llama; the reference's projections take the first as a flag,
src/llmserve/model/llama.py:64-66) give the projections bias vectors ``*_proj.bias``: such a layer
runs its products and the bias sums as kernels of their own, not the fused decode kernels.

The position encoding is a part of its own.  One whose ``rotary_layout`` is ``"half"`` (pairs
``(j, j + head_dim/2)`` over the whole head, angles tabulated as ``rotary_table``) is applied by the
kernels that also store keys and values; any other is asked to ``apply`` itself to q and k.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import Mixer, PagedKVSpec, PartSpec, TensorSpec, build_part, register_part


class PagedAttention(Mixer):
    def __init__(
        self,
        hidden_size: int,
        num_heads: int,
        num_kv_heads: int,
        head_dim: int,
        scale: float,
        window: int | None = None,
        position: PartSpec | None = None,
        own_kv: bool = True,
        qkv_bias: bool = False,
        out_bias: bool = False,
    ):
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads {num_heads} is not a multiple of num_kv_heads {num_kv_heads}")
        if window is not None and window < 1:
            raise ValueError(f"window must be positive or None, got {window}")
        if not 1 <= int(head_dim) <= 256:
            raise ValueError(f"head_dim {head_dim} is not supported: the attention kernels take head sizes up to 256")
        self.hidden_size = int(hidden_size)
        self.num_heads = int(num_heads)
        self.num_kv_heads = int(num_kv_heads)
        self.head_dim = int(head_dim)
        self.scale = float(scale)
        self.window = None if window is None else int(window)
        self.own_kv = bool(own_kv)
        self.qkv_bias = bool(qkv_bias)
        self.out_bias = bool(out_bias)
        self.b_in: torch.Tensor | None = None  # [(H + 2 KV) D] with qkv_bias
        self.b_out: torch.Tensor | None = None  # [hidden] with out_bias
        self.position = build_part("position", position) if position is not None else None
        self.w_in: torch.Tensor | None = None  # [(H + 2 KV) D, hidden], or [H D, hidden] without own_kv
        self.w_out: torch.Tensor | None = None  # [hidden, H D]

    def tensors(self) -> dict[str, TensorSpec]:
        q = self.num_heads * self.head_dim
        kv = self.num_kv_heads * self.head_dim
        specs = {"q_proj.weight": TensorSpec((q, self.hidden_size))}
        if self.own_kv:
            specs["k_proj.weight"] = TensorSpec((kv, self.hidden_size))
            specs["v_proj.weight"] = TensorSpec((kv, self.hidden_size))
        specs["o_proj.weight"] = TensorSpec((self.hidden_size, q))
        if self.qkv_bias:
            specs["q_proj.bias"] = TensorSpec((q,))
            if self.own_kv:
                specs["k_proj.bias"] = TensorSpec((kv,))
                specs["v_proj.bias"] = TensorSpec((kv,))
        if self.out_bias:
            specs["o_proj.bias"] = TensorSpec((self.hidden_size,))
        return specs

    def bind(self, tensors, dtype, device) -> None:
        names = ["q_proj.weight"] + (["k_proj.weight", "v_proj.weight"] if self.own_kv else [])
        fused = torch.cat([tensors[n].to(dtype) for n in names], dim=0)
        self.w_in = fused.to(device).contiguous()
        self.w_out = tensors["o_proj.weight"].to(device=device, dtype=dtype).contiguous()
        if self.qkv_bias:
            self.b_in = torch.cat([tensors[n.replace(".weight", ".bias")].to(dtype) for n in names]).to(device).contiguous()
        if self.out_bias:
            self.b_out = tensors["o_proj.bias"].to(device=device, dtype=dtype).contiguous()
        if self.position is not None:
            self.position.bind({}, dtype, device)

    def cache_spec(self) -> PagedKVSpec:
        return PagedKVSpec(self.num_kv_heads, self.head_dim, self.window)

    accepts_sink = True

    @property
    def graph_safe(self) -> bool:
        """The same launches whatever a step holds, if the position encoding's are too."""
        return self.position is None or bool(getattr(self.position, "graph_safe", False))

    def _rotary_table(self):
        """The table of a position encoding that the fused kernels know how to apply, else None."""
        if getattr(self.position, "rotary_layout", None) != "half":
            return None
        table = getattr(self.position, "rotary_table", None)
        return table if table is not None and table.shape[1] == self.head_dim else None

    def forward(self, x, ctx, cache, sink=None):
        H, KV, D = self.num_heads, self.num_kv_heads, self.head_dim
        table = self._rotary_table()
        qkv = None
        if (self.position is None or table is not None) and self.b_in is None:
            # few rows: projection, rotation and the cache write in one kernel
            qkv = ops.linear_qkv_rope(
                x, self.w_in, ctx.positions, table, cache.slot_map, cache.pool, H, KV, D, write_kv=self.own_kv
            )
        if qkv is None:
            qkv = self._project_rotate_store(x, ctx, cache, table)
        out = ops.paged_attention(
            qkv,
            cache.pool,
            cache.page_table,
            ctx,
            num_heads=H,
            num_kv_heads=KV,
            head_dim=D,
            scale=self.scale,
            window=self.window,
        )
        # the contribution to the 32-bit residual stream leaves the product in 32-bit: it is the sum's largest addend
        if self.b_out is not None:
            return ops.add_bias(ops.linear(out, self.w_out, out_dtype=torch.float32), self.b_out.float())
        if sink is not None:
            handed_on = sink.linear(out, self.w_out)
            if handed_on is not None:
                return handed_on
        return ops.linear(out, self.w_out, out_dtype=torch.float32)

    def _project_rotate_store(self, x, ctx, cache, table):
        H, KV, D = self.num_heads, self.num_kv_heads, self.head_dim
        qkv = ops.linear(x, self.w_in)
        if self.b_in is not None:
            ops.add_bias(qkv, self.b_in)
        if self.position is not None and table is None:
            # a position encoding without a table: let it rewrite q and k, then store unrotated
            n = qkv.shape[0]
            q = qkv[:, : H * D].unflatten(1, (H, D))
            k = qkv[:, H * D : (H + KV) * D].unflatten(1, (KV, D)) if self.own_kv else qkv.new_empty((n, 0, D))
            self.position.apply(q, k, ctx.positions)
        ops.rope_kv_write(
            qkv, ctx.positions, table, cache.slot_map, cache.pool, H, KV, D, write_kv=self.own_kv
        )
        return qkv


register_part("mixer", "attention", PagedAttention)
