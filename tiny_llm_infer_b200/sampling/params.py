"""Per-request sampling options, with the reference's names, defaults and checks
(engine/include/sampling_params.h:10-34): ``max_tokens`` 64, ``temperature`` 0 (at most
1e-6 means greedy), ``top_p`` 1 in (0, 1], ``ignore_eos`` false, ``seed`` 0 (0 means: use
the request id).  The reference has no top-k, penalties or stop strings; nor has this."""
from __future__ import annotations

from dataclasses import dataclass

GREEDY_BELOW = 1.0e-6


@dataclass
class SamplingParams:
    max_tokens: int = 64
    temperature: float = 0.0
    top_p: float = 1.0
    ignore_eos: bool = False
    seed: int = 0

    def validate(self) -> None:
        if self.max_tokens < 0:
            raise ValueError(f"max_tokens is {self.max_tokens}; it cannot be negative")
        if self.temperature < 0.0:
            raise ValueError(f"temperature is {self.temperature}; it cannot be negative")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError(f"top_p is {self.top_p}; it must lie in (0, 1]")

    @property
    def greedy(self) -> bool:
        return not self.temperature > GREEDY_BELOW
