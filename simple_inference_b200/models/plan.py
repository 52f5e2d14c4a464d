"""A model as data: parts chosen layer by layer, and the order layers run in.

An architecture module turns its typed configuration into a ``ModelPlan``:
the embedding (a registered kind), a list of ``LayerPlan`` (each a block
``PartSpec`` plus the checkpoint name of every tensor it needs), the run order, the
final norm and the output head (a registered kind too).  ``DecoderModel`` builds the parts through the registries,
binds the loaded tensors and executes the plan for a step; it knows nothing of
any particular architecture.

The run order is a list of ``RunStep``.  A step names a layer (a layer may be
named more than once: the same weights run again, each run with a cache entry
of its own) and the cache entry it uses; ``writes_cache=False`` lets a run read
the entry another run filled instead of storing its own keys and values.

The reference fixes all of this in code: 28 identical ``TransformerBlock``s run
in index order (``model/llama.py:92-106,174-186``).
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..parts.base import Block, CacheSpec, LayerCache, PartSpec, Runtime, StepPlanner, TensorSpec
from ..parts.registry import BLOCKS, EMBEDDINGS, HEADS, NORMS


@dataclass
class LayerPlan:
    block: PartSpec
    # part-local tensor name ("mixer.wq") -> name in the checkpoint
    tensor_names: dict[str, str]


@dataclass(frozen=True)
class RunStep:
    layer: int
    cache_entry: int
    writes_cache: bool = True


@dataclass
class ModelPlan:
    hidden_size: int
    vocab_size: int
    layers: list[LayerPlan]
    run_order: list[RunStep]
    final_norm: PartSpec
    tie_embeddings: bool
    embedding_names: dict[str, str]      # embedding-local tensor name -> name in the checkpoint
    final_norm_names: dict[str, str]
    head_names: dict[str, str]           # tensors of the head (not needed when it is tied)
    max_positions: int
    eos_token_ids: tuple[int, ...] = ()
    bos_token_id: int | None = None
    embedding: PartSpec | None = None    # default: the plain lookup ``token_embedding``
    head: PartSpec | None = None         # default: ``linear_head``, tied as ``tie_embeddings`` says

    def embedding_spec(self) -> PartSpec:
        return self.embedding or PartSpec("token_embedding", {
            "vocab_size": self.vocab_size, "hidden_size": self.hidden_size})

    def head_spec(self) -> PartSpec:
        return self.head or PartSpec("linear_head", {
            "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
            "tied": self.tie_embeddings})

    @staticmethod
    def sequential(num_layers: int) -> list[RunStep]:
        return [RunStep(i, i, True) for i in range(num_layers)]


@dataclass
class CacheEntryInfo:
    """Cache need of one cache entry of the run order."""
    spec: CacheSpec | None
    writer: int | None = None  # index into run_order of the run that fills it


class DecoderModel:
    """Executes a ``ModelPlan``: embedding, blocks in run order, final norm, head."""

    def __init__(self, plan: ModelPlan):
        self.plan = plan
        self.embedding = EMBEDDINGS.build(plan.embedding_spec())
        self.blocks: list[Block] = [BLOCKS.build(lp.block) for lp in plan.layers]
        self.final_norm = NORMS.build(plan.final_norm)
        self.head = HEADS.build(plan.head_spec())
        self.rt: Runtime | None = None
        self._check_run_order()

    # ------------------------------------------------------------ structure
    def _check_run_order(self) -> None:
        n_layers = len(self.blocks)
        entries: dict[int, CacheEntryInfo] = {}
        for idx, step in enumerate(self.plan.run_order):
            if not (0 <= step.layer < n_layers):
                raise ValueError(f"run order names layer {step.layer}, the model has {n_layers}")
            spec = self.blocks[step.layer].mixer.cache_spec()
            info = entries.get(step.cache_entry)
            if info is None:
                if not step.writes_cache and spec is not None:
                    raise ValueError(f"run {idx} reads cache entry {step.cache_entry} "
                                     f"before any run has written it")
                entries[step.cache_entry] = CacheEntryInfo(spec, idx)
            else:
                if step.writes_cache:
                    raise ValueError(f"runs {info.writer} and {idx} both write cache entry "
                                     f"{step.cache_entry}")
                if info.spec != spec:
                    raise ValueError(f"run {idx} reads cache entry {step.cache_entry} whose "
                                     f"shape {info.spec} differs from its own {spec}")
        if sorted(entries) != list(range(len(entries))):
            raise ValueError("cache entries of the run order must be numbered 0..n-1")
        self.cache_entries = [entries[i] for i in range(len(entries))]

    def cache_specs(self) -> list[CacheSpec | None]:
        """Cache need of every cache entry, in entry order (for the cache manager)."""
        return [e.spec for e in self.cache_entries]

    def tensor_specs(self) -> dict[str, TensorSpec]:
        """Checkpoint tensor name -> spec, for the loader and the random-weights writer."""
        out: dict[str, TensorSpec] = {}
        for local, spec in self.embedding.tensors().items():
            out[self.plan.embedding_names[local]] = spec
        for lp, block in zip(self.plan.layers, self.blocks):
            for local, spec in block.tensors().items():
                out[lp.tensor_names[local]] = spec
        for local, spec in self.final_norm.tensors().items():
            out[self.plan.final_norm_names[local]] = spec
        for local, spec in self.head.tensors().items():
            out[self.plan.head_names[local]] = spec
        return out

    def step_planners(self) -> dict[str, type[StepPlanner]]:
        """The step planner classes the model's parts ask for, one per name."""
        out: dict[str, type[StepPlanner]] = {}
        for part in (self.embedding, *self.blocks, self.final_norm, self.head):
            for planner in part.step_planners():
                out.setdefault(planner.name, planner)
        return out

    def optional_tensor_names(self) -> set[str]:
        """Names a checkpoint may carry that the model does not need."""
        if self.plan.tie_embeddings:  # a tied checkpoint may still store the head
            return set(self.plan.head_names.values()) - set(self.tensor_specs())
        return set()

    # -------------------------------------------------------------- weights
    def bind(self, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        """``tensors``: checkpoint name -> device tensor in its final dtype."""
        self.rt = rt
        self.embedding.bind({local: tensors[name]
                             for local, name in self.plan.embedding_names.items()}, rt)
        for lp, block in zip(self.plan.layers, self.blocks):
            block.bind({local: tensors[name] for local, name in lp.tensor_names.items()}, rt)
        self.final_norm.bind({local: tensors[name]
                              for local, name in self.plan.final_norm_names.items()}, rt)
        self.head.bind({local: tensors[self.plan.head_names[local]]
                        for local in self.head.tensors()}, rt, embedding=self.embedding)

    # ----------------------------------------------------------------- step
    def forward(self, ctx, caches: list[LayerCache | None]) -> torch.Tensor:
        """Run the tokens of ``ctx``; return float32 logits at ``ctx.logit_rows``.

        ``caches[e]`` is the view of cache entry ``e``.
        """
        residual = self.embedding.forward(ctx.token_ids, ctx)
        delta = None
        order = self.plan.run_order
        for i, step in enumerate(order):
            # who adds this block's output to the residual stream: the next block's first norm,
            # or the final norm
            taker = self.blocks[order[i + 1].layer].first_norm() if i + 1 < len(order) \
                else self.final_norm
            ctx.next_takes_partial_sums = bool(taker is not None and taker.takes_partial_sums)
            cache = caches[step.cache_entry]
            if cache is not None and cache.writes != step.writes_cache:
                cache = LayerCache(cache.spec, cache.group, cache.pool, cache.state,
                                   cache.page_size, step.writes_cache)
            delta = self.blocks[step.layer].forward(residual, delta, ctx, cache)
        if ctx.num_logit_rows == 0:
            return ctx.ws.get("logits", (0, self.plan.vocab_size), torch.float32,
                              row_cap=ctx.ws.max_logit_rows)
        h = self.final_norm.add_forward(residual, delta, ctx, rows=ctx.logit_rows, tag="final_norm")
        return self.head.forward(h, ctx)
