"""The step function: run a batch of (request, its next tokens) from the cache.

``ModelRunner.step`` takes portions of prompts beside single decoded tokens,
cut anywhere, makes room for them in the cache, runs only those tokens as one
flat batch and returns float32 logits at the wanted places.  It is the merger
of the reference's two runners (``serving/prefill.py:60-76`` for whole prompt
suffixes, ``serving/paged_decoder.py:363-408`` for one token per request),
which the reference runs as two separate forwards per step.

A decode-only batch (one token and one wanted row per request) can be replayed
from a CUDA graph captured per batch-size bucket (reference
``model/cuda_graph.py:62-88``, buckets ``serving/paged_decoder.py:93-106``);
rows that pad a bucket read and write only the scratch page and scratch slot.
"""

from __future__ import annotations

from typing import Hashable

import torch

from ..cache.manager import CacheManager
from ..models.plan import DecoderModel
from ..parts.base import Runtime
from .batch import BatchBuilder, StepContext, StepEntry, Workspace


def decode_buckets(max_seqs: int) -> list[int]:
    """Powers of two below ``max_seqs``, then ``max_seqs`` itself."""
    out, b = [], 1
    while b < max_seqs:
        out.append(b)
        b *= 2
    out.append(max_seqs)
    return out


class ModelRunner:
    def __init__(self, model: DecoderModel, cache: CacheManager, rt: Runtime, max_step_tokens: int,
                 max_seqs: int, max_seq_len: int, cuda_graphs: bool = False,
                 max_logit_rows: int | None = None):
        if model.rt is None:
            raise RuntimeError("the model has no weights bound")
        self.model = model
        self.cache = cache
        self.rt = rt
        self.max_step_tokens = max_step_tokens
        self.max_seqs = max_seqs
        self.max_seq_len = max_seq_len
        self.ws = Workspace(rt.device, max_step_tokens,
                            max_logit_rows if max_logit_rows is not None else max_seqs)
        self.builder = BatchBuilder(cache, max_step_tokens, max_seqs, max_seq_len, rt.device,
                                    planners=model.step_planners())
        self.layer_caches = cache.layer_caches()
        self.cuda_graphs = cuda_graphs and rt.device.type == "cuda"
        self._graphs: dict[int, tuple[torch.cuda.CUDAGraph, torch.Tensor]] = {}
        self._graph_kernels: dict[int, int] = {}   # bucket -> kernels of this package in its graph
        self._logit_rows: dict[tuple[int, int], torch.Tensor] = {}
        self.replayed_kernels = 0                  # kernels launched through graph replays so far
        self._buckets = decode_buckets(max_seqs)
        self.last_context: StepContext | None = None

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self, entries: list[StepEntry]) -> torch.Tensor:
        """Run ``entries`` as one batch; returns ``[wanted, vocab]`` float32 logits.

        Every request must have been admitted to the cache.  The rows of the
        result follow the order of the entries and of each entry's ``want``.
        The returned tensor is a view of a buffer the next step overwrites.
        """
        if not entries:
            raise ValueError("a step needs at least one entry")
        seen: set[Hashable] = set()
        for e in entries:
            if e.request in seen:
                raise ValueError(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
            if not e.tokens:
                raise ValueError(f"request {e.request!r} brings no tokens")
        starts = [self.cache.extend(e.request, len(e.tokens)) for e in entries]

        decode_only = all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries)
        if self.cuda_graphs and decode_only:
            return self._replay(entries, starts)
        ctx = self.builder.build(entries, starts, self.ws)
        self.last_context = ctx
        return self.model.forward(ctx, self.layer_caches)

    # ---------------------------------------------------------------- graphs
    def bucket_for(self, n: int) -> int:
        for b in self._buckets:
            if b >= n:
                return b
        raise ValueError(f"{n} sequences exceed max_seqs {self.max_seqs}")

    def _fixed_context(self, entries: list[StepEntry], starts: list[int], bucket: int) -> StepContext:
        ctx = self.builder.build(entries, starts, self.ws, pad_to=bucket)
        # Inside a graph every size is the bucket's and launch shapes are planned
        # for the longest context the engine allows; kernels read the true
        # lengths from device memory.
        ctx.fixed_shape = True
        ctx.max_kv_len = self.max_seq_len
        return ctx

    def _replay(self, entries: list[StepEntry], starts: list[int]) -> torch.Tensor:
        bucket = self.bucket_for(len(entries))
        if bucket not in self._graphs:   # first met inside a live step: capture on padding rows
            self._capture(bucket)
        ctx = self._fixed_context(entries, starts, bucket)
        self.last_context = ctx
        graph, logits = self._graphs[bucket]
        graph.replay()
        self.replayed_kernels += self._graph_kernels[bucket]
        rows = self._logit_rows.get((bucket, len(entries)))
        if rows is None:   # a view per (bucket, live rows), made once
            rows = self._logit_rows[(bucket, len(entries))] = logits[:len(entries)]
        return rows

    def _capture(self, bucket: int) -> None:
        """Warm up on a side stream, then record one forward (reference model/cuda_graph.py:62-88).

        Always on padding rows alone: they read and write only the scratch page and the
        scratch slot, so neither the warm-up runs nor the recording touch what a live request
        holds.  (Running a live step several times would be harmless for keys and values,
        which land in the same slots each time, but not for a mixer that advances a state.)
        """
        ctx = self._fixed_context([], [], bucket)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self.model.forward(ctx, self.layer_caches)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.ws.freeze()
        from .. import ops
        graph = torch.cuda.CUDAGraph()
        before = ops.launch_count
        with torch.cuda.graph(graph):
            logits = self.model.forward(ctx, self.layer_caches)
        self._graph_kernels[bucket] = ops.launch_count - before
        ops.launch_count = before  # recorded, not run
        self._graphs[bucket] = (graph, logits)

    def capture_all(self) -> None:
        """Capture the decode graph of every bucket ahead of time."""
        if not self.cuda_graphs:
            return
        for bucket in self._buckets:
            if bucket not in self._graphs:
                self._capture(bucket)
