"""Options of one request, with the reference's names and meanings
(src/llmserve/datatypes.py:6-13)."""

from __future__ import annotations

from dataclasses import dataclass


@dataclass
class SamplingParams:
    temperature: float = 0.0  # <= 0 means greedy
    top_k: int = 0  # 0 disables
    top_p: float = 1.0  # 1.0 disables
    max_new_tokens: int = 128
    eos_token_id: int | None = None
    seed: int | None = None  # None: a fresh seed per request

    def __post_init__(self) -> None:
        if self.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be >= 1")
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0")
        if not 0.0 <= self.top_p <= 1.0:
            raise ValueError("top_p must lie in [0, 1]")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0
