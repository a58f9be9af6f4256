"""The flat description of one step that every part reads.

The reference pads every sequence of a forward pass to the longest
(src/llmserve/kvcache/paged.py:181-218: positions, valid, write slots, tables, lengths, last
index, each ``[B, T]`` or ``[B]``).  Here a step is flat: the new tokens of all requests lie end
to end, request r owning ``cu_tokens[r]:cu_tokens[r+1]``; nothing is padded, and a portion of
a prompt sits beside single decoded tokens.  All integer arrays travel in one pinned buffer
and one copy to the device.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch


@dataclass
class StepEntry:
    """The next tokens of one request, and the places among them whose logits are wanted."""

    request: object
    tokens: list[int]
    want: list[int] = field(default_factory=list)


@dataclass
class StepContext:
    num_tokens: int
    num_requests: int
    num_logits: int
    token_ids: torch.Tensor  # [N] int32
    positions: torch.Tensor  # [N] int32, absolute position of each token in its request
    token_request: torch.Tensor  # [N] int32, index into the step's requests
    cu_tokens: torch.Tensor  # [R + 1] int32
    context_lens: torch.Tensor  # [R] int32, tokens each request holds after this step
    logit_rows: torch.Tensor  # [P] int32, rows of the flat batch whose logits are returned
    state_slots: torch.Tensor  # [R] int32
    # host copies, for grid sizes and for parts that walk requests on the host
    host_cu_tokens: list[int]
    host_context_lens: list[int]
    host_state_slots: list[int]
    max_query_len: int
    max_context_len: int
    # True for the fixed buffers of a captured decode step: one token per request, every row's logits wanted,
    # the same addresses at every replay (a model may then build a plan for the step once and keep it)
    static_decode: bool = False


def pack_step(entries: list[StepEntry], lengths: list[int], state_slots: np.ndarray, group_arrays, device):
    """Build the :class:`StepContext` and the device copies of each group's page table and slot
    map.  ``lengths[r]`` is what request r held before the step."""
    counts = [len(e.tokens) for e in entries]
    n, r = sum(counts), len(entries)
    cu = np.zeros(r + 1, dtype=np.int32)
    cu[1:] = np.cumsum(counts)
    token_ids = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries]).astype(np.int32)
    positions = np.concatenate([np.arange(s, s + c, dtype=np.int32) for s, c in zip(lengths, counts)])
    token_request = np.repeat(np.arange(r, dtype=np.int32), counts)
    ctx_lens = np.asarray([s + c for s, c in zip(lengths, counts)], dtype=np.int32)
    rows = []
    for i, e in enumerate(entries):
        for w in e.want:
            if not 0 <= w < counts[i]:
                raise ValueError(f"request {e.request!r} wants place {w} among {counts[i]} tokens")
            rows.append(int(cu[i]) + w)
    logit_rows = np.asarray(rows, dtype=np.int32)

    pieces = [token_ids, positions, token_request, cu, ctx_lens, logit_rows, state_slots.astype(np.int32)]
    for table, slot_map in group_arrays:
        pieces += [table.reshape(-1), slot_map]
    # every piece starts on a 16-byte boundary (4 int32) so kernels may read them with wide loads
    offsets, total = [], 0
    for p in pieces:
        offsets.append(total)
        total += -(-p.size // 4) * 4
    host = torch.empty(max(total, 4), dtype=torch.int32, pin_memory=(torch.device(device).type == "cuda"))
    host_np = host.numpy()
    for p, off in zip(pieces, offsets):
        host_np[off : off + p.size] = p
    dev = host.to(device, non_blocking=True)

    def piece(i):
        return dev[offsets[i] : offsets[i] + pieces[i].size]

    ctx = StepContext(
        num_tokens=n,
        num_requests=r,
        num_logits=len(rows),
        token_ids=piece(0),
        positions=piece(1),
        token_request=piece(2),
        cu_tokens=piece(3),
        context_lens=piece(4),
        logit_rows=piece(5),
        state_slots=piece(6),
        host_cu_tokens=cu.tolist(),
        host_context_lens=ctx_lens.tolist(),
        host_state_slots=state_slots.tolist(),
        max_query_len=max(counts),
        max_context_len=int(ctx_lens.max()),
    )
    group_tensors = []
    for g, (table, _) in enumerate(group_arrays):
        group_tensors.append((piece(7 + 2 * g).view(table.shape), piece(8 + 2 * g)))
    return ctx, group_tensors, (host.numel() * 4)
