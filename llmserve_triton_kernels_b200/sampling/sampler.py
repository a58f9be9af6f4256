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


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)
        self.d2h_bytes = 0
        self.h2d_bytes = 0

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
            # one buffer, one copy: [temperature | top_k | top_p | - | seeds (64-bit) | counters (64-bit)]
            packed = np.zeros(8 * rows, dtype=np.int32)
            packed[0:rows] = np.asarray([p.temperature for p in params], dtype=np.float32).view(np.int32)
            packed[rows : 2 * rows] = np.asarray([p.top_k for p in params], dtype=np.int32)
            packed[2 * rows : 3 * rows] = np.asarray([p.top_p for p in params], dtype=np.float32).view(np.int32)
            packed[4 * rows : 6 * rows] = np.asarray(seeds, dtype=np.uint64).view(np.int32)
            packed[6 * rows : 8 * rows] = np.asarray(counters, dtype=np.uint64).view(np.int32)
            host = torch.from_numpy(packed)
            if self.device.type == "cuda":
                host = host.pin_memory()
            dev = host.to(self.device, non_blocking=True)
            self.h2d_bytes = packed.nbytes
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
