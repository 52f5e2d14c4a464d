"""Sampling options of a request, with the reference's names and meanings.

``temperature`` 0 is greedy (top-k and top-p ignored), 1 leaves the logits
alone, negative is an error (reference ``sampling.py:39-52,159-160``);
``top_k`` <= 0 or >= vocabulary is off (``:68-83``); ``top_p`` >= 1 is off,
<= 0 keeps the top token (``:95-128``).  ``seed`` is new: the reference draws
from torch's global generator (``:169-172``); here a request's draws depend on
(seed, request stream, index of the token) only.
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    seed: int = 0

    def __post_init__(self) -> None:
        if self.temperature < 0:
            raise ValueError(f"temperature must be >= 0 (got {self.temperature}); 0 is greedy")
        if not (self.top_p == self.top_p):
            raise ValueError("top_p is NaN")
