"""Per-request sampling settings, with the reference's names, defaults and limits
(python/instinct/sampling.py:19-41)."""

from __future__ import annotations

import math
from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0  # 0 picks the most likely token
    top_p: float = 1.0  # keep a token while the probability mass before it is below top_p
    top_k: int = 0  # 0 = off; 1 = greedy
    min_p: float = 0.0  # keep tokens at least min_p times as likely as the most likely one
    seed: int | None = None  # fixes the request's draws whatever else is in the batch

    def __post_init__(self) -> None:
        if not (isinstance(self.temperature, (int, float)) and math.isfinite(self.temperature) and 0.0 <= self.temperature <= 10.0):
            raise ValueError("temperature must be between 0 and 10")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1]")
        if type(self.top_k) is not int or self.top_k < 0:
            raise ValueError("top_k must be a non-negative integer")
        if not 0.0 <= self.min_p < 1.0:
            raise ValueError("min_p must be in [0, 1)")
        if self.seed is not None and type(self.seed) is not int:
            raise ValueError("seed must be an integer")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0 or self.top_k == 1


GREEDY = SamplingParams()
