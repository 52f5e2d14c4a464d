"""A request: the unit of work that lives across many steps.

Lifecycle as in the reference (``serving/request.py:41-92``):
WAITING (queued) -> PREFILL (admitted, prompt not yet wholly processed) ->
DECODE (one token per step) -> FINISHED.  New here: ``prefilled`` counts the
prompt tokens already run, because a prompt may be processed in portions.
"""

from __future__ import annotations

import enum
import itertools
from dataclasses import dataclass, field

from ..sampling.params import SamplingParams


class RequestState(enum.Enum):
    WAITING = "waiting"
    PREFILL = "prefill"
    DECODE = "decode"
    FINISHED = "finished"


_ids = itertools.count(1)


@dataclass
class Request:
    prompt_tokens: list[int]
    max_new_tokens: int
    sampling: SamplingParams = field(default_factory=SamplingParams)
    id: int = field(default_factory=lambda: next(_ids))
    stream: int = 0                # sampling stream: separates the draws of requests that share a seed
    state: RequestState = RequestState.WAITING
    slot: int | None = None        # admission slot = row of per-request state
    prefilled: int = 0             # prompt tokens already run
    pos: int = 0                   # tokens in the cache = position of the next token
    generated: list[int] = field(default_factory=list)
    eos_hit: bool = False
    finish_reason: str | None = None   # "stop" (end token) or "length"

    @property
    def prompt_len(self) -> int:
        return len(self.prompt_tokens)

    @property
    def num_generated(self) -> int:
        return len(self.generated)

    @property
    def last_token(self) -> int:
        return self.generated[-1] if self.generated else self.prompt_tokens[-1]

    def should_finish(self) -> bool:
        return self.eos_hit or self.num_generated >= self.max_new_tokens
