"""Scheduler: admits requests, cuts prompts into portions, plans each step.

Admission follows the reference's ``Scheduler.admit`` (``serving/scheduler.py:
93-123``): first come first served; a request is admitted while a slot is free,
the sum of context lengths of the running set stays within ``token_budget``
(one request is always let in when nothing runs), and ``can_admit`` (the page
reservation) agrees.  When the head of the queue cannot reserve its pages it
waits and everything behind it waits too: nothing skips ahead (``:109-113``).

Planning a step is new (the reference runs whole prompts, ``plan.md:833-848``
only sketches portions): every request in DECODE gets one token; then requests
in PREFILL, oldest first, get ``min(chunk_size, rest of the prompt, rest of
the step's token budget)`` tokens.  A request draws its first token in the step
that runs the last token of its prompt.

What happens when pages run out: they cannot run out in mid-flight.  A request
reserves pages for ``prompt + max_new_tokens`` when it is admitted and is not
admitted before that many are free; a request that could never fit is refused
when it is added.  There is no preemption, swapping or recomputation.
"""

from __future__ import annotations

from collections import deque
from collections.abc import Callable

from .request import Request, RequestState


class Scheduler:
    def __init__(self, max_running: int, max_tokens_per_step: int, chunk_size: int | None = None,
                 token_budget: int | None = None):
        if max_running <= 0:
            raise ValueError("max_running must be positive")
        if max_tokens_per_step < max_running:
            raise ValueError(f"max_tokens_per_step {max_tokens_per_step} cannot hold one token "
                             f"for each of {max_running} running requests")
        self.max_running = max_running
        self.max_tokens_per_step = max_tokens_per_step
        self.chunk_size = chunk_size if chunk_size else max_tokens_per_step
        if self.chunk_size <= 0:
            raise ValueError("chunk_size must be positive")
        self.token_budget = token_budget
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []

    def add(self, req: Request) -> None:
        req.state = RequestState.WAITING
        self.waiting.append(req)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def evict_finished(self) -> list[Request]:
        done = [r for r in self.running if r.state is RequestState.FINISHED]
        if done:
            self.running = [r for r in self.running if r.state is not RequestState.FINISHED]
        return done

    def _running_tokens(self) -> int:
        return sum(r.prompt_len + r.num_generated for r in self.running)

    def admit(self, can_admit: Callable[[Request], bool],
              on_admit: Callable[[Request], None]) -> list[Request]:
        """Move requests from WAITING to PREFILL while slots, budget and pages allow."""
        admitted: list[Request] = []
        used = self._running_tokens()
        while self.waiting and len(self.running) < self.max_running:
            nxt = self.waiting[0]
            if self.token_budget is not None and (self.running or admitted):
                if used + nxt.prompt_len > self.token_budget:
                    break
            if not can_admit(nxt):
                break  # the head waits for pages; nobody behind it jumps the queue
            self.waiting.popleft()
            on_admit(nxt)
            nxt.state = RequestState.PREFILL
            nxt.prefilled = 0
            nxt.pos = 0
            self.running.append(nxt)
            admitted.append(nxt)
            used += nxt.prompt_len
        return admitted

    def plan_step(self) -> list[tuple[Request, int]]:
        """(request, number of its next tokens to run) for this step."""
        plan: list[tuple[Request, int]] = []
        budget = self.max_tokens_per_step
        for r in self.running:
            if r.state is RequestState.DECODE:
                plan.append((r, 1))
                budget -= 1
        for r in self.running:
            if r.state is RequestState.PREFILL and budget > 0:
                n = min(self.chunk_size, r.prompt_len - r.prefilled, budget)
                if n > 0:
                    plan.append((r, n))
                    budget -= n
        return plan
