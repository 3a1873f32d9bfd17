"""Per-request sampling settings.

The field names, defaults and allowed ranges are the request schema of the reference
(python/instinct/sampling.py:19-41), so that its callers' settings carry over. The ranges
live in one table, :data:`RANGES`; the C++ scheduler holds the same table
(``sampling_ranges()`` of the host module) and checks every submitted request against it
again, and a test compares the two.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, fields
from typing import NamedTuple


class Range(NamedTuple):
    """The interval a numeric setting must lie in; ``whole`` asks for a Python int."""

    low: float
    high: float
    low_open: bool = False
    high_open: bool = False
    whole: bool = False

    def holds(self, value: object) -> bool:
        if self.whole and type(value) is not int:
            return False
        if isinstance(value, bool) or not isinstance(value, (int, float)) or math.isnan(value):
            return False
        above = value > self.low if self.low_open else value >= self.low
        below = value < self.high if self.high_open else value <= self.high
        return above and below

    def __str__(self) -> str:
        text = f"{'(' if self.low_open else '['}{self.low:g}, {self.high:g}{')' if self.high_open else ']'}"
        return ("a whole number in " if self.whole else "a number in ") + text


RANGES: dict[str, Range] = {
    "temperature": Range(0.0, 10.0),  # 0 takes the most likely token
    "top_p": Range(0.0, 1.0, low_open=True),  # tokens stay while the mass ahead of them is below top_p
    "top_k": Range(0, float(2**31 - 1), whole=True),  # 0 switches the filter off, 1 is greedy
    "min_p": Range(0.0, 1.0, high_open=True),  # tokens stay if at least min_p times as likely as the best
}


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    min_p: float = 0.0
    seed: int | None = None  # pins the request's draws, whatever shares its batch

    def __post_init__(self) -> None:
        broken = [
            f"{f.name}={getattr(self, f.name)!r} is not {RANGES[f.name]}"
            for f in fields(self)
            if f.name in RANGES and not RANGES[f.name].holds(getattr(self, f.name))
        ]
        if self.seed is not None and type(self.seed) is not int:
            broken.append(f"seed={self.seed!r} is neither None nor an int")
        if broken:
            raise ValueError("sampling settings refused: " + "; ".join(broken))

    @property
    def greedy(self) -> bool:
        """No draw is needed: zero temperature, or a top-k of one."""
        return self.top_k == 1 or self.temperature == 0.0


GREEDY = SamplingParams()
