"""Next tokens for the rows of a step, chosen on the device.

Parity: src/llmserve/sampling/sampler.py:16-39 (greedy when temperature <= 0; otherwise
temperature, top-k, top-p, then a draw) and src/llmserve/scheduler/engine.py:279-285 (one
argmax and one host read for an all-greedy batch).  The draw differs in its random numbers
only: instead of a generator object per request, row i uses the uniform number of
``(seed_i, number of tokens request i has drawn before)``, so a request's tokens do not depend on
what else is in the batch or on preemption.
"""

from __future__ import annotations

import numpy as np
import torch

from .. import ops
from .params import SamplingParams


class _ParameterBuffers:
    """Where the parameters of one batch size travel: four pinned host buffers used in turn (each taken again only
    after the kernel that fetched it last has ended) and their one place on the device."""

    TURNS = 4

    def __init__(self, rows: int, device: torch.device):
        self.on_device = torch.zeros(8 * rows, dtype=torch.int32, device=device)
        self.rows, self.pinned, self.turn = rows, [], 0

    def take(self):
        """(array to fill, the same as a pinned tensor, event to record once its fetch has been launched)."""
        if len(self.pinned) < self.TURNS:
            tensor = torch.zeros(8 * self.rows, dtype=torch.int32, pin_memory=True)
            self.pinned.append((tensor.numpy(), tensor, torch.cuda.Event()))
            return self.pinned[-1]
        array, tensor, fetched = self.pinned[self.turn % self.TURNS]
        self.turn += 1
        fetched.synchronize()
        return array, tensor, fetched


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)
        self.d2h_bytes = 0
        self.h2d_bytes = 0
        self._buffers: dict[int, _ParameterBuffers] = {}  # by number of rows

    def _parameters(self, rows: int):
        """Buffers for the rows' parameters: (array to fill, the same as a pinned tensor, its place on the device,
        event).  On a CUDA device a kernel brings the pinned buffer to the device (no hand-over to the copy engine; the
        sampling kernel itself does not read host memory: every small read is a trip over the bus of its own, and
        they queue up)."""
        if self.device.type != "cuda":
            packed = np.zeros(8 * rows, dtype=np.int32)
            return packed, None, torch.from_numpy(packed), None
        buffers = self._buffers.get(rows)
        if buffers is None:
            buffers = self._buffers[rows] = _ParameterBuffers(rows, self.device)
        packed, tensor, fetched = buffers.take()
        return packed, tensor, buffers.on_device, fetched

    def __call__(self, logits: torch.Tensor, params: list[SamplingParams], seeds: list[int], counters: list[int]) -> list[int]:
        """``logits [rows, vocab]`` float32 on the device -> one token id per row, on the host."""
        if logits.shape[0] == 0:
            return []
        return self.on_device(logits, params, seeds, counters).tolist()

    def on_device(self, logits: torch.Tensor, params: list[SamplingParams], seeds: list[int], counters: list[int],
                  host_out: torch.Tensor | None = None) -> torch.Tensor:
        """The same, but the token ids stay on the device (int32 ``[rows]``): the next step can be fed from there
        before the host has seen them.  ``host_out`` (int32 ``[rows]``, pinned host memory) gets them too, written by
        the kernel, and may be read once the stream has passed this point."""
        rows = logits.shape[0]
        self.h2d_bytes = 0
        extra = {} if host_out is None else {"host_out": host_out}
        if all(p.greedy for p in params):
            tokens = ops.argmax(logits, **extra)
        else:
            # one buffer: [temperature | top_k | top_p | - | seeds (64-bit) | counters (64-bit)]
            packed, host, dev, fetched = self._parameters(rows)
            packed[0:rows] = np.asarray([p.temperature for p in params], dtype=np.float32).view(np.int32)
            packed[rows : 2 * rows] = np.asarray([p.top_k for p in params], dtype=np.int32)
            packed[2 * rows : 3 * rows] = np.asarray([p.top_p for p in params], dtype=np.float32).view(np.int32)
            packed[4 * rows : 6 * rows] = np.asarray(seeds, dtype=np.uint64).view(np.int32)
            packed[6 * rows : 8 * rows] = np.asarray(counters, dtype=np.uint64).view(np.int32)
            self.h2d_bytes = packed.nbytes
            if host is not None:
                ops.fetch_words(host, dev)
                fetched.record()
            tokens = ops.sample(
                logits,
                dev[0:rows].view(torch.float32),
                dev[rows : 2 * rows],
                dev[2 * rows : 3 * rows].view(torch.float32),
                dev[4 * rows : 6 * rows].view(torch.int64),
                dev[6 * rows : 8 * rows].view(torch.int64),
                **extra,
            )
        self.d2h_bytes = rows * 4
        return tokens
