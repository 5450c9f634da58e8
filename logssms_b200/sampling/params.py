"""Per-request sampling options, with the reference's names, defaults and greedy rule
(python/logssms/core.py:31-41), plus a seed."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_k: int = -1
    top_p: float = 1.0
    ignore_eos: bool = False
    max_tokens: int = 1024
    seed: int | None = None        # None: drawn from the sampler's own seed and the request's number

    @property
    def is_greedy(self) -> bool:
        return (self.temperature <= 0.0 or self.top_k == 1) and self.top_p == 1.0
