"""A runnable model built from a :class:`ModelPlan`: the same class for every architecture.

It owns the token table, the layers (blocks of parts), the final norm and the output matrix,
declares every tensor it expects by checkpoint name, and runs one step over a flat batch of
tokens.  Parity for the order of operations: src/llmserve/model/llama.py:155-185 (embedding,
the layers in order, gather of the wanted rows *before* the final norm, output matrix).
"""

from __future__ import annotations

import torch

from .. import ops
from ..parts.base import Block, PagedKVSpec, StateSpec, TensorSpec, build_part
from .plan import ModelPlan


class Model:
    def __init__(self, plan: ModelPlan, dtype: torch.dtype, device: torch.device | str):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"compute dtype must be bfloat16 or float32, got {dtype}")
        self.plan = plan
        self.dtype = dtype
        self.device = torch.device(device)
        self.blocks: list[Block] = []
        self._named_parts: list[tuple[str, object]] = []  # (prefix, part) of every tensor-owning part
        for spec in plan.layers:
            parts = {}
            for role, category in (
                ("mixer_norm", "norm"),
                ("mixer", "mixer"),
                ("ff_norm", "norm"),
                ("feed_forward", "feed_forward"),
            ):
                part_spec = getattr(spec, role)
                parts[role] = build_part(category, part_spec)
                self._named_parts.append((part_spec.prefix, parts[role]))
            block = build_part("block", type(spec.block)(spec.block.kind, {**spec.block.params, **parts}, spec.block.prefix))
            self._named_parts.append((spec.block.prefix, block))
            self.blocks.append(block)
        self.final_norm = build_part("norm", plan.final_norm)
        self._named_parts.append((plan.final_norm.prefix, self.final_norm))
        self.embedding: torch.Tensor | None = None
        self.head: torch.Tensor | None = None

    # ------------------------------------------------------------------ tensors
    def tensor_specs(self) -> dict[str, TensorSpec]:
        """Every tensor of the checkpoint by its full name."""
        plan = self.plan
        specs = {plan.embedding: TensorSpec((plan.vocab_size, plan.hidden_size))}
        for prefix, part in self._named_parts:
            for local, spec in part.tensors().items():
                name = prefix + local
                if name in specs:
                    raise ValueError(f"two parts claim the tensor {name!r}")
                specs[name] = spec
        if plan.head is not None:
            specs[plan.head] = TensorSpec((plan.vocab_size, plan.hidden_size))
        return specs

    def ignored_tensor_names(self) -> set[str]:
        """Names a checkpoint may carry that the model does not read (a copy of a tied output matrix)."""
        return {"lm_head.weight"} if self.plan.head is None else set()

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        plan = self.plan
        self.embedding = tensors[plan.embedding].to(device=self.device, dtype=self.dtype).contiguous()
        if plan.head is None:
            self.head = self.embedding
        else:
            self.head = tensors[plan.head].to(device=self.device, dtype=self.dtype).contiguous()
        for prefix, part in self._named_parts:
            local = {name: tensors[prefix + name] for name in part.tensors()}
            part.bind(local, self.dtype, self.device)
        if self.dtype == torch.bfloat16:
            # the order in which a step streams its matrices, for the decode products' L2 prefetch
            order = []
            for run in self.plan.schedule:
                block = self.blocks[run.layer]
                for part in (getattr(block, "mixer", None), getattr(block, "feed_forward", None)):
                    order += list(getattr(part, "streamed_weights", lambda: [])())
            ops.set_weight_order(order + [self.head])

    def weight_bytes(self) -> int:
        """Bytes of every distinct weight tensor a step reads (the token table only if it is also the head)."""
        seen: dict[int, int] = {}

        def visit(obj):
            for value in vars(obj).values():
                if isinstance(value, torch.Tensor):
                    seen[value.data_ptr()] = value.numel() * value.element_size()
                elif hasattr(value, "bind") and hasattr(value, "tensors"):
                    visit(value)

        for _, part in self._named_parts:
            visit(part)
        seen[self.head.data_ptr()] = self.head.numel() * self.head.element_size()
        return sum(seen.values())

    @property
    def graph_safe(self) -> bool:
        """Every part launches the same kernels whatever the step's contents, so a decode step can be captured."""
        return all(
            getattr(b, "graph_safe", False) for b in self.blocks
        ) and getattr(self.final_norm, "graph_safe", False)

    def _fused_decode(self, ctx, caches):
        """A captured decode step of few tokens through the one-kernel path, when every layer of the
        order is of the kind that kernel runs and all agree in their sizes; else None."""
        plan = getattr(ctx, "_fused_plan", None)
        if plan is None:
            plan = self._make_fused_plan(ctx, caches) or False
            ctx._fused_plan = plan
        return ops.fused_decode_run(plan) if plan else None

    def _make_fused_plan(self, ctx, caches):
        order = self.plan.schedule
        if any(run.cache_of is not None for run in order) or getattr(self.final_norm, "fused_params", None) is None:
            return None
        specs = []
        for i, run in enumerate(order):
            spec = getattr(self.blocks[run.layer], "fused_decode_spec", lambda c: None)(caches[i])
            if spec is None:
                return None
            specs.append(spec)
        first = specs[0]
        if any(s["dims"] != first["dims"] or s["rotary_table"] is not first["rotary_table"] or s["page_size"] != first["page_size"] for s in specs):
            return None
        layers = []
        for i, s in enumerate(specs):
            nxt = specs[i + 1]["mixer_norm"] if i + 1 < len(specs) else self.final_norm.fused_params()
            layers.append({**s, "next_norm": nxt})
        hidden, heads, kv_heads, head_dim, inter = first["dims"]
        return ops.fused_decode_plan(
            ctx=ctx, hidden=hidden, num_heads=heads, num_kv_heads=kv_heads, head_dim=head_dim, inter=inter,
            vocab=self.plan.vocab_size, page_size=first["page_size"], embedding=self.embedding, first_norm=first["mixer_norm"],
            rotary_table=first["rotary_table"], layers=layers, head=self.head,
        )

    # ------------------------------------------------------------------ caches
    def cache_specs(self) -> list[PagedKVSpec | StateSpec | None]:
        """For each entry of the order: what its mixer keeps, or None if it keeps nothing of its
        own (no cache, or it reads an earlier entry's)."""
        out = []
        for run in self.plan.schedule:
            out.append(None if run.cache_of is not None else self.blocks[run.layer].mixer.cache_spec())
        return out

    # ------------------------------------------------------------------ step
    def forward(self, ctx, caches) -> torch.Tensor:
        """Run the tokens of ``ctx`` through every entry of the order; ``caches[i]`` is the view
        of entry i's cache.  Returns 32-bit logits ``[len(ctx.logit_rows), vocab]``."""
        if getattr(ctx, "static_decode", False) and self.dtype == torch.bfloat16:
            logits = self._fused_decode(ctx, caches)
            if logits is not None:
                return logits
        resid = ops.embed(ctx.token_ids, self.embedding)
        pending = None
        order = self.plan.schedule
        for i, run in enumerate(order):
            # the norm that meets the stream next, so that a block's last product may prepare for it
            next_norm = self.blocks[order[i + 1].layer].mixer_norm if i + 1 < len(order) else None
            pending = self.blocks[run.layer].forward(resid, pending, ctx, caches[i], next_norm=next_norm)
        if ctx.num_logits == 0:
            return torch.empty((0, self.plan.vocab_size), dtype=torch.float32, device=self.device)
        x = self.final_norm.add_forward(resid, pending, rows=ctx.logit_rows)
        return ops.linear(x, self.head, out_dtype=torch.float32)
