"""Sampling settings of one request: names, defaults and ranges as in flyweight
(src/flyweight/sampling.py:11-47): temperature 0.8, top_k 40, top_p 0.95, min_p 0.05,
penalties off with a 64-token window; ``seed`` None means "pick one"."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class SamplingConfig:
    temperature: float = 0.8
    top_k: int = 40
    top_p: float = 0.95
    min_p: float = 0.05
    seed: Optional[int] = None
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    penalty_window: int = 64

    def __post_init__(self) -> None:
        if self.temperature < 0:
            raise ValueError("temperature must be non-negative")
        if self.top_k < 0:
            raise ValueError("top_k must be non-negative")
        if not 0 < self.top_p <= 1:
            raise ValueError("top_p must be in (0, 1]")
        if not 0 <= self.min_p <= 1:
            raise ValueError("min_p must be in [0, 1]")
        if not 1.0 <= self.repetition_penalty <= 2.0:
            raise ValueError("repetition_penalty must be in [1, 2]")
        if not -2.0 <= self.presence_penalty <= 2.0:
            raise ValueError("presence_penalty must be in [-2, 2]")
        if not -2.0 <= self.frequency_penalty <= 2.0:
            raise ValueError("frequency_penalty must be in [-2, 2]")
        if not 0 <= self.penalty_window <= 256:
            raise ValueError("penalty_window must be in [0, 256]")

    @property
    def penalizes(self) -> bool:
        return self.penalty_window > 0 and (self.repetition_penalty != 1.0
                                            or self.presence_penalty != 0.0
                                            or self.frequency_penalty != 0.0)

    @property
    def greedy(self) -> bool:
        """Argmax of the raw logits decides (temperature 0 or a single candidate, and no
        penalty that could demote it)."""
        return (self.temperature <= 0.0 or self.top_k == 1) and not self.penalizes


GREEDY = SamplingConfig(temperature=0.0, top_k=1, top_p=1.0, min_p=0.0)
