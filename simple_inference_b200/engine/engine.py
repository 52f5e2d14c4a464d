"""The inference engine: requests in, tokens out, continuous batching in between.

``InferenceEngine`` keeps the reference's public face
(``serving/engine.py:95-517``): the constructor's option names, and
``add_request(prompt_tokens, max_new_tokens) -> Request``,
``step() -> {request id: token}``, ``run() -> {request id: Request}``,
``has_work()``, ``reset()``, ``warmup()``.  Underneath, one step is ONE batch:
a token for every request that is decoding beside portions of the prompts of
requests that are still prefilling (the reference runs a padded prompt batch
and a decode batch as two forwards, ``:314-349``, and never cuts a prompt).

Options the reference does not have: ``max_tokens_per_step`` and ``chunk_size``
(how prompts are cut), ``seed`` (sampling is reproducible per request), and
per-request sampling options on ``add_request``.
"""

from __future__ import annotations

import time
from collections.abc import Iterator
from pathlib import Path
from typing import Any

import torch

from ..cache.manager import CacheManager, pages_for
from ..models.load import load_model, random_model
from ..models.plan import DecoderModel
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .batch import StepEntry
from .request import Request, RequestState
from .runner import ModelRunner
from .scheduler import Scheduler


class InferenceEngine:
    def __init__(
        self,
        model: DecoderModel,
        max_running: int,
        max_seq_len: int,
        block_size: int = 16,
        num_kv_blocks: int | None = None,
        token_budget: int | None = None,
        eos_id: int | None = None,
        temperature: float = 0.0,
        top_k: int = 0,
        top_p: float = 1.0,
        warmup: bool = True,
        use_cuda_graphs: bool = True,
        max_tokens_per_step: int | None = None,
        chunk_size: int | None = None,
        seed: int = 0,
    ):
        """
        model:          a ``DecoderModel`` with weights bound (``load_model`` / ``random_model``).
        max_running:    most requests admitted at a time.
        max_seq_len:    most tokens (prompt + generated) of one request.
        block_size:     tokens per cache page.
        num_kv_blocks:  pages per layer group; default ``max_running * ceil(max_seq_len /
                        block_size)`` as in the reference (``serving/engine.py:180-183``).
        token_budget:   soft cap on the summed context of the running set (admission).
        eos_id:         stop token; default: the configuration's; -1: never stop.
        temperature, top_k, top_p: default sampling options (temperature 0 = greedy).
        warmup:         capture the decode graphs at construction.
        use_cuda_graphs: replay decode-only steps from CUDA graphs.
        max_tokens_per_step: most tokens one step runs (default ``max(max_running, 2048)``).
        chunk_size:     longest portion of one prompt in one step (default: no extra cut).
        seed:           default sampling seed.
        """
        if model.rt is None:
            raise RuntimeError("the model has no weights bound")
        if block_size <= 0:
            raise ValueError(f"block_size must be positive, got {block_size}")
        if max_seq_len > model.plan.max_positions:
            raise ValueError(f"max_seq_len {max_seq_len} exceeds the model's "
                             f"max_position_embeddings {model.plan.max_positions}")
        self.model = model
        self.rt = model.rt
        self.max_running = max_running
        self.max_seq_len = max_seq_len
        self.block_size = block_size
        if eos_id is None:
            self.eos_ids: tuple[int, ...] = tuple(model.plan.eos_token_ids)
        else:
            self.eos_ids = () if eos_id < 0 else (eos_id,)
        self.defaults = SamplingParams(temperature, top_k, top_p, seed)
        self.max_tokens_per_step = max_tokens_per_step or max(max_running, 2048)
        self.num_kv_blocks = (num_kv_blocks if num_kv_blocks is not None
                              else max_running * pages_for(max_seq_len, block_size))
        # by default every group gets enough pages of its own size for max_running full requests
        pool_pages = (num_kv_blocks if num_kv_blocks is not None
                      else lambda page: max_running * pages_for(max_seq_len, page))

        self.scheduler = Scheduler(max_running, self.max_tokens_per_step, chunk_size, token_budget)
        self.cache = CacheManager(model.cache_specs(), block_size, pool_pages, max_running,
                                  self.max_tokens_per_step, dtype=self.rt.dtype,
                                  device=self.rt.device)
        self.runner = ModelRunner(model, self.cache, self.rt, self.max_tokens_per_step,
                                  max_running, max_seq_len, cuda_graphs=use_cuda_graphs)
        self.sampler = Sampler(self.rt.device, max_running)
        self.use_cuda_graphs = self.runner.cuda_graphs
        self.steps = 0
        self._arrivals = 0
        if warmup:
            self.warmup()

    # ----------------------------------------------------------- construction
    @classmethod
    def from_folder(cls, model_dir: str | Path, dtype: str = "bfloat16", device: str = "cuda",
                    **options: Any) -> "InferenceEngine":
        _, model = load_model(model_dir, dtype, device)
        return cls(model, **options)

    @classmethod
    def from_random(cls, config: dict[str, Any], seed: int = 0, dtype: str = "bfloat16",
                    device: str = "cuda", **options: Any) -> "InferenceEngine":
        _, model = random_model(config, seed, dtype, device)
        return cls(model, **options)

    # ------------------------------------------------------------- public API
    def add_request(self, prompt_tokens: list[int], max_new_tokens: int,
                    sampling: SamplingParams | None = None) -> Request:
        """Queue a request (checks as the reference's, ``serving/engine.py:228-254``)."""
        if not prompt_tokens:
            raise ValueError("prompt_tokens is empty")
        if max_new_tokens < 1:
            raise ValueError(f"max_new_tokens must be >= 1 (got {max_new_tokens})")
        total = len(prompt_tokens) + max_new_tokens
        if total > self.max_seq_len:
            raise ValueError(f"prompt_len ({len(prompt_tokens)}) + max_new_tokens "
                             f"({max_new_tokens}) > max_seq_len ({self.max_seq_len})")
        if not self.cache.fits_at_all(total):
            raise ValueError(f"request needs more cache pages than the whole pool of "
                             f"{self.num_kv_blocks} pages of {self.block_size} tokens")
        vocab = self.model.plan.vocab_size
        if any((not isinstance(t, int)) or t < 0 or t >= vocab for t in prompt_tokens):
            raise ValueError("prompt contains token ids outside the vocabulary")
        # Requests that take the engine's default options draw from streams of their
        # own (their order of arrival); explicit options mean exactly what they say.
        stream = 0
        if sampling is None:
            self._arrivals += 1
            stream = self._arrivals
        req = Request(list(prompt_tokens), max_new_tokens, sampling or self.defaults, stream=stream)
        self.scheduler.add(req)
        return req

    def has_work(self) -> bool:
        return self.scheduler.has_work()

    def reset(self) -> None:
        """Drop every queued and running request and give all pages and slots back."""
        for r in self.scheduler.running:
            if self.cache.is_admitted(r.id):
                self.cache.release(r.id)
        self.scheduler.waiting.clear()
        self.scheduler.running.clear()

    def warmup(self) -> None:
        """Compile what this model needs and capture the decode graphs, on padding rows only."""
        self.runner.capture_all()
        if self.rt.device.type == "cuda":
            torch.cuda.synchronize(self.rt.device)

    def step(self) -> dict[int, int]:
        """One iteration: free finished requests, admit, run one batch, sample.

        Returns ``{request id: new token}`` for every request that drew a token.
        """
        for r in self.scheduler.evict_finished():
            self.cache.release(r.id)
        self.scheduler.admit(
            can_admit=lambda r: self.cache.can_admit(r.prompt_len + r.max_new_tokens),
            on_admit=self._on_admit)
        plan = self.scheduler.plan_step()
        if not plan:
            return {}
        entries: list[StepEntry] = []
        drawing: list[Request] = []
        for r, n in plan:
            if r.state is RequestState.DECODE:
                entries.append(StepEntry(r.id, [r.last_token], [0]))
                drawing.append(r)
            else:
                tokens = r.prompt_tokens[r.prefilled:r.prefilled + n]
                last = r.prefilled + n == r.prompt_len
                entries.append(StepEntry(r.id, tokens, [n - 1] if last else []))
                if last:
                    drawing.append(r)
        logits = self.runner.step(entries)
        tokens_out = self.sampler.sample(
            logits, [(r.sampling, r.stream, r.num_generated) for r in drawing]) if drawing else []
        for r, n in plan:
            r.pos += n
            if r.state is RequestState.PREFILL:
                r.prefilled += n
        emitted: dict[int, int] = {}
        for r, tok in zip(drawing, tokens_out):
            r.generated.append(tok)
            emitted[r.id] = tok
            if tok in self.eos_ids:
                r.eos_hit = True
            if r.should_finish():
                r.state = RequestState.FINISHED
                r.finish_reason = "stop" if r.eos_hit else "length"
            else:
                r.state = RequestState.DECODE
        self.steps += 1
        return emitted

    def _on_admit(self, r: Request) -> None:
        r.slot = self.cache.admit(r.id, r.prompt_len + r.max_new_tokens)

    def run(self) -> dict[int, Request]:
        """Step until every queued request has finished; returns them by id."""
        seen: dict[int, Request] = {r.id: r for r in self.scheduler.waiting}
        seen.update({r.id: r for r in self.scheduler.running})
        while self.has_work():
            self.step()
        # the last finished requests still hold pages until the next eviction
        for r in self.scheduler.evict_finished():
            self.cache.release(r.id)
        return seen

    # ------------------------------------------------------ single-request use
    def generate(self, prompt_tokens: list[int], max_new_tokens: int = 256,
                 temperature: float | None = None, top_k: int | None = None,
                 top_p: float | None = None, seed: int | None = None) -> Iterator[int]:
        """Yield the tokens of one request as they are drawn.

        The counterpart of the reference's ``generate()`` (``generate.py:50-119``)
        on token ids; unlike it, the first drawn token is yielded too.
        """
        d = self.defaults
        sp = SamplingParams(d.temperature if temperature is None else temperature,
                            d.top_k if top_k is None else top_k,
                            d.top_p if top_p is None else top_p,
                            d.seed if seed is None else seed)
        req = self.add_request(prompt_tokens, max_new_tokens, sp)
        while req.state is not RequestState.FINISHED:
            out = self.step()
            if req.id in out:
                yield out[req.id]

    def generate_with_stats(self, prompt_tokens: list[int], max_new_tokens: int = 256,
                            on_token=None, **sampling: Any) -> tuple[list[int], dict[str, float]]:
        """Tokens of one request and the reference's timing record (``generate.py:132-237``)."""
        cuda = self.rt.device.type == "cuda"
        if cuda:
            torch.cuda.reset_peak_memory_stats(self.rt.device)
            torch.cuda.synchronize()
        start = time.perf_counter()
        stamps: list[float] = []
        out: list[int] = []
        for tok in self.generate(prompt_tokens, max_new_tokens, **sampling):
            out.append(tok)
            stamps.append(time.perf_counter())
            if on_token is not None:
                on_token(tok)
        wall = time.perf_counter() - start
        ttft = (stamps[0] - start) if stamps else wall
        gaps = [b - a for a, b in zip(stamps, stamps[1:])]
        tpot = sum(gaps) / len(gaps) if gaps else 0.0
        n_prompt = len(prompt_tokens)
        stats = {
            "prompt_tokens": n_prompt,
            "new_tokens": len(out),
            "ttft_ms": round(ttft * 1e3, 2),
            "tpot_ms": round(tpot * 1e3, 3),
            "prefill_ms": round(ttft * 1e3, 2),
            "decode_tok_s": round(1.0 / tpot, 1) if tpot > 0 else 0.0,
            "total_wall_ms": round(wall * 1e3, 2),
            "total_tok_s": round((n_prompt + len(out)) / wall, 1) if wall > 0 else 0.0,
            "peak_vram_gb": round(torch.cuda.max_memory_allocated(self.rt.device) / 1e9, 2)
            if cuda else 0.0,
        }
        return out, stats
