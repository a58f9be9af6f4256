"""Steps as CUDA graphs.

A step whose shape has been seen before — how many tokens each request brings and which of them want
logits — launches the same kernels with the same grids every time, so the whole pass (some hundred and
fifty launches for 22 layers) is captured once per shape and replayed.  Only the step's integer arrays
change: they are written into a pinned buffer of fixed layout and brought to the device in one piece
before the replay.  Decode steps (one token per request) are captured at their first occurrence; other
shapes (a prompt of 512 tokens, eight of them side by side, a portion beside decoded tokens) at their
second, and the least recently used are dropped beyond a limit.  The reference notes launch and host
overhead as its next bottleneck and CUDA graphs as the cure (its docs/PROFILING.md:19-20 and the closing
notes of its design document) but does not build them.

Page tables have the model's full width in a graph (``ceil(max_positions / page_size)``), and
``StepContext.max_context_len`` is the model's limit, so no launch depends on how long the requests
are at the time.  The graphs of one step function share one memory pool: they never run at the same
time, and what one keeps between replays (its logits) is never freed.
"""

from __future__ import annotations

import numpy as np
import torch

from .. import ops
from .batch import StepContext


def _pad4(n: int) -> int:
    return -(-n // 4) * 4


class StepGraph:
    def __init__(self, model, cache, counts: tuple[int, ...], wants: tuple[tuple[int, ...], ...], owner=None):
        """``counts[r]``: tokens that request r of the step brings; ``wants[r]``: the places among them whose
        logits are returned.  ``owner``: whoever keeps the graphs (an object with an attribute ``graph_pool``): the
        graphs of one owner share one memory pool, that of the first one captured."""
        self.model, self.cache, self.owner = model, cache, owner
        self.counts, self.wants = tuple(counts), tuple(tuple(w) for w in wants)
        R, N = len(self.counts), sum(self.counts)
        self.R, self.N = R, N
        cu = np.zeros(R + 1, dtype=np.int32)
        cu[1:] = np.cumsum(self.counts)
        rows = [int(cu[r]) + w for r, want in enumerate(self.wants) for w in want]
        for r, want in enumerate(self.wants):
            for w in want:
                if not 0 <= w < self.counts[r]:
                    raise ValueError(f"place {w} is wanted among {self.counts[r]} tokens")
        P = len(rows)
        self.widths = [-(-model.plan.max_positions // g.page_size) for g in cache.groups]
        sizes = [N, N, N, R + 1, R, P, R]  # ids, positions, token_request, cu, ctx_lens, logit_rows, state_slots
        for w in self.widths:
            sizes += [R * w, N]
        self.offsets = np.concatenate(([0], np.cumsum([_pad4(s) for s in sizes]))).tolist()
        self.sizes = sizes
        total = self.offsets[-1]
        self.host = torch.zeros(total, dtype=torch.int32, pin_memory=True)
        self.host_np = self.host.numpy()
        self.dev = torch.zeros(total, dtype=torch.int32, device=cache.device)
        self._counts_np = np.asarray(self.counts, dtype=np.int64)
        self._within = np.arange(N, dtype=np.int64) - np.repeat(cu[:-1].astype(np.int64), self._counts_np)
        self._piece_np(2)[:] = np.repeat(np.arange(R, dtype=np.int32), self._counts_np)
        self._piece_np(3)[:] = cu
        self._piece_np(5)[:] = rows
        self.copied = torch.cuda.Event()
        self.graph: torch.cuda.CUDAGraph | None = None
        self.logits: torch.Tensor | None = None
        self.launches = 0
        self.decode_only = all(c == 1 for c in self.counts) and all(w == (0,) for w in self.wants)
        d = self._piece
        self.ctx = StepContext(
            num_tokens=N, num_requests=R, num_logits=P,
            token_ids=d(0), positions=d(1), token_request=d(2), cu_tokens=d(3), context_lens=d(4), logit_rows=d(5),
            state_slots=d(6), host_cu_tokens=cu.tolist(), host_context_lens=None, host_state_slots=None,
            max_query_len=max(self.counts), max_context_len=model.plan.max_positions, static_decode=self.decode_only,
        )
        group_tensors = []
        for g, w in enumerate(self.widths):
            group_tensors.append((d(7 + 2 * g).view(R, w), d(8 + 2 * g)))
        self.views = cache.views(group_tensors, self.ctx.state_slots, None)
        self.h2d_bytes = total * 4

    def _piece(self, i: int) -> torch.Tensor:
        return self.dev[self.offsets[i] : self.offsets[i] + self.sizes[i]]

    def _piece_np(self, i: int) -> np.ndarray:
        return self.host_np[self.offsets[i] : self.offsets[i] + self.sizes[i]]

    def fill(self, tokens, lengths: list[int], state_slots: np.ndarray, group_arrays) -> None:
        """Write the step's arrays into the pinned buffer and start their way to the device.  ``tokens``: the ids
        of all requests end to end on the host, or (decode steps) an int32 tensor ``[R]`` on the device (the step
        before has put its choices there and the host has not seen them yet), which takes the place of the host's
        token ids on the way.  ``lengths[r]``: what request r held before the step."""
        self.copied.synchronize()  # the previous copy has left the pinned buffer
        R = self.R
        on_device = isinstance(tokens, torch.Tensor)
        starts = np.asarray(lengths, dtype=np.int64)
        self._piece_np(0)[:] = 0 if on_device else tokens
        self._piece_np(1)[:] = np.repeat(starts, self._counts_np) + self._within
        self._piece_np(4)[:] = starts + self._counts_np
        self._piece_np(6)[:] = state_slots
        for g, (table, slot_map) in enumerate(group_arrays):
            dst = self._piece_np(7 + 2 * g).reshape(R, self.widths[g])
            dst[:, : table.shape[1]] = table
            self._piece_np(8 + 2 * g)[:] = slot_map
        # a kernel that reads the pinned buffer (shorter than a copy by the copy engine) and takes the token ids
        # from the device where they are there
        ops.fetch_words(self.host, self.dev, tokens if on_device else None)
        self.copied.record()

    def run(self) -> torch.Tensor:
        """Logits ``[wanted places, vocab]`` of the step whose arrays were filled last.  The tensor is the graph's
        own from the second call on: the next replay overwrites it.  The first call runs the step once, kernel by
        kernel (which also sets up libraries and kernel attributes, as must happen outside a capture), hands out
        that pass's logits and then only records the graph, which executes nothing: no step runs twice, so a part
        that keeps state of its own need not be idempotent to be captured."""
        if self.graph is None:
            return self._first_run_and_capture()
        self.graph.replay()
        ops.add_launches(self.launches)
        return self.logits

    def _first_run_and_capture(self) -> torch.Tensor:
        current = torch.cuda.current_stream()
        side = torch.cuda.Stream()
        side.wait_stream(current)
        with torch.cuda.stream(side):
            first = self.model.forward(self.ctx, self.views)
        current.wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        before = ops.launch_count()
        pool = getattr(self.owner, "graph_pool", None)
        with torch.cuda.graph(graph, pool=pool):
            self.logits = self.model.forward(self.ctx, self.views)
        if self.owner is not None and pool is None:
            self.owner.graph_pool = graph.pool()
        self.launches = ops.launch_count() - before
        ops.add_launches(-self.launches)  # a capture launches nothing
        self.graph = graph
        return first


class DecodeGraph(StepGraph):
    """The graph of a decode step of ``num_requests`` requests: one token each, its logits wanted."""

    def __init__(self, model, cache, num_requests: int, owner=None):
        super().__init__(model, cache, (1,) * int(num_requests), ((0,),) * int(num_requests), owner)
