"""A runnable model built from a :class:`ModelPlan`: the same class for every architecture.

It owns the token table, the layers (blocks of parts), the final norm and the output matrix,
declares every tensor it expects by checkpoint name, and runs one step over a flat batch of
tokens.  Parity for the order of operations: src/llmserve/model/llama.py:155-185 (embedding,
the layers in order, gather of the wanted rows *before* the final norm, output matrix).
"""

from __future__ import annotations

import torch

from .. import ops
from ..parts.base import Block, PagedKVSpec, StateSpec, TensorSpec, build_part, part_factory
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
        for i, spec in enumerate(plan.layers):
            factory = part_factory("block", spec.block.kind)
            roles = getattr(factory, "roles", None)
            if not roles:
                raise ValueError(f"block kind {spec.block.kind!r} declares no roles (Block.roles: role -> part category)")
            if set(roles) != set(spec.parts):
                raise ValueError(
                    f"layer {i}: block kind {spec.block.kind!r} is built from {sorted(roles)}, the plan gives {sorted(spec.parts)}"
                )
            parts = {}
            for role, category in roles.items():
                parts[role] = build_part(category, spec.parts[role])
                self._named_parts.append((spec.parts[role].prefix, parts[role]))
            block = build_part("block", spec.block, **parts)
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
        """Names a checkpoint may carry that the model does not read; the plan lists them."""
        return set(self.plan.ignored)

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

    # ------------------------------------------------------------------ caches
    def cache_specs(self) -> list[PagedKVSpec | StateSpec | None]:
        """For each entry of the order: what its mixer keeps, or None if it keeps nothing of its
        own (no cache, or it reads an earlier entry's)."""
        out = []
        for run in self.plan.schedule:
            out.append(None if run.cache_of is not None else self.blocks[run.layer].cache_spec())
        return out

    # ------------------------------------------------------------------ step
    def forward(self, ctx, caches) -> torch.Tensor:
        """Run the tokens of ``ctx`` through every entry of the order; ``caches[i]`` is the view
        of entry i's cache.  Returns 32-bit logits ``[len(ctx.logit_rows), vocab]``."""
        if ops.checked():
            self._check_step(ctx, caches)
        resid = self.embed_tokens(ctx)
        pending = None
        order = self.plan.schedule
        for i, run in enumerate(order):
            # the norm that meets the stream next, so that a block's last product may prepare for it
            next_norm = self.blocks[order[i + 1].layer].first_norm() if i + 1 < len(order) else None
            pending = self.blocks[run.layer].forward(resid, pending, ctx, caches[i], next_norm=next_norm)
        if ctx.num_logits == 0:
            return torch.empty((0, self.plan.vocab_size), dtype=torch.float32, device=self.device)
        x = self.final_norm.add_forward(resid, pending, rows=ctx.logit_rows)
        return self.project_logits(x)

    def _check_step(self, ctx, caches) -> None:
        """Checked mode: the step's arrays are looked over on the device before any kernel indexes with them."""
        slots = next((c.states.shape[0] for c in caches if hasattr(c, "states")), 0)
        ops.check_step_arrays(ctx, self.plan.vocab_size, self.plan.max_positions, slots)
        seen = []
        for c in caches:
            if hasattr(c, "page_table") and all(c.page_table.data_ptr() != t.data_ptr() for t in seen):
                ops.check_page_group(ctx, c.page_table, c.slot_map, c.page_size, c.pool.shape[0], c.spec.window, len(seen))
                seen.append(c.page_table)

    def embed_tokens(self, ctx) -> torch.Tensor:
        """The residual stream that the first layer meets: the tokens' rows of the table, in 32-bit ``[N, hidden]``.
        An architecture that scales or otherwise prepares its embeddings overrides this in a subclass that it names
        when it registers (``register_architecture(..., model_class=...)``)."""
        return ops.embed(ctx.token_ids, self.embedding)

    def project_logits(self, x) -> torch.Tensor:
        """32-bit logits ``[rows, vocab]`` of the normalised rows ``x`` (a tensor, or the factored form that the
        last block handed on).  The place for an architecture's cap or scale of its logits, in a subclass."""
        return ops.linear(x, self.head, out_dtype=torch.float32)
