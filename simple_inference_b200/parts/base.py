"""Interfaces of the parts a model is put together from.

A model is a list of blocks; a block arranges a *mixer* (attention here), a
*feed-forward* and their *norms*; a mixer may use a *position encoding*.  Each
part takes its sizes and constants as constructor parameters, declares the
tensors it needs (``tensors``) and the cache it needs (``cache_spec``), and is
given its loaded tensors once (``bind``).  No part knows which model it is in:
the architecture module translates a config.json into ``PartSpec`` records
(kind name + parameters) layer by layer, and the registries in
``parts/registry.py`` turn those into objects.

The reference builds the same pieces as ``nn.Module``s with constructor
constants (``model/block.py:56-99``, ``ops/attention.py:70-103``,
``ops/mlp.py:61-88``, ``ops/rmsnorm.py:49-53``, ``ops/rope.py:72-118``) but
hard-wires their kinds; here the kinds are data.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import TYPE_CHECKING, Any

import torch

if TYPE_CHECKING:  # pragma: no cover
    from ..engine.batch import StepContext


# --------------------------------------------------------------------------
# Declarations: tensors and caches
# --------------------------------------------------------------------------

@dataclass(frozen=True)
class TensorSpec:
    """One tensor a part needs from the checkpoint.

    kind:
      ``matrix``  operand of a matrix product; held in the compute dtype
                  (bfloat16 when serving, float32 on the 32-bit path).
      ``vector``  gains and other small tensors; bfloat16 stays bfloat16, a
                  tensor stored in 32-bit stays 32-bit (on the 32-bit path
                  everything is float32).
      ``table``   integer table, held as int32.
    init: how the random-weights mode fills it (``normal``: N(0, std);
      ``gain``: 1 + N(0, gain_std); ``zeros``).
    """

    shape: tuple[int, ...]
    kind: str = "matrix"
    init: str = "normal"


@dataclass(frozen=True)
class PagedKVSpec:
    """Keys and values per token, kept in pages.

    ``window`` None keeps every key; an integer w lets a query at position p see
    keys in (p - w, p] only, so pages wholly before that range are given back.
    ``page_size`` None takes the cache manager's page size; a number gives this
    kind of cache pages of its own size.
    """

    num_kv_heads: int
    head_dim: int
    window: int | None = None
    page_size: int | None = None

    storage = "pages"

    def page_shape(self, page_size: int) -> tuple[int, ...]:
        """One page of one cache entry: keys then values, ``[2, kv_heads, page_size, head_dim]``."""
        return (2, self.num_kv_heads, page_size, self.head_dim)


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size (one row per admission slot)."""

    shape: tuple[int, ...]
    dtype: str = "float32"

    storage = "slots"

    def slot_shape(self) -> tuple[int, ...]:
        return tuple(self.shape)


# What a mixer may return from ``cache_spec()``.  The cache manager knows two ways of
# storing: ``storage == "pages"`` (memory that grows with the request: the spec says how one
# page of ``page_size`` tokens is shaped, ``page_shape(page_size)``, which page size it wants,
# ``page_size`` or None, and whether old pages may go, ``window``) and ``storage == "slots"``
# (one row of ``slot_shape()`` per request).  Specs that compare equal share a group of pages.
# Any frozen dataclass with these attributes will do; the two above are the built-in ones.
CacheSpec = PagedKVSpec | StateSpec


@dataclass
class LayerCache:
    """What one run of a layer sees of the cache.

    For a spec stored in pages: ``pool`` is ``[pages+1, *spec.page_shape(page_size)]``
    (for ``PagedKVSpec`` ``[pages+1, 2, kv_heads, page_size, head_dim]``, index 0/1 of
    the second axis = keys/values; the last page is scratch), ``group`` selects this
    layer group's block tables and write slots in the ``StepContext``.  For a spec
    stored in slots: ``state`` is ``[slots+1, *spec.slot_shape()]``, row = the
    request's slot, the last row is scratch.
    ``writes`` is False when the layer only reads a cache that another layer
    filled.
    """

    spec: CacheSpec
    group: int = 0
    pool: torch.Tensor | None = None
    state: torch.Tensor | None = None
    page_size: int = 0
    writes: bool = True


@dataclass
class Runtime:
    """Where and in which precision the parts run."""

    device: torch.device
    dtype: torch.dtype  # activations, matrices and caches: bfloat16 or float32

    @property
    def is_fp32(self) -> bool:
        return self.dtype == torch.float32


# --------------------------------------------------------------------------
# Part interfaces
# --------------------------------------------------------------------------

class Part:
    """Common base: declares tensors, receives them, runs on the device."""

    def tensors(self) -> dict[str, TensorSpec]:
        return {}

    def bind(self, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        """Take ownership of the loaded tensors (already on device, right dtype)."""
        self.rt = rt

    def step_planners(self) -> list[type["StepPlanner"]]:
        """Classes of the host-side planners this part (or the parts inside it) wants run once
        per step; every batch builder makes its own instance of each."""
        return []


class StepPlanner:
    """Host work a kind of part needs once per step, whatever the number of layers of that kind.

    The batch builder makes one instance per ``name`` and gives it a segment of the step's
    description buffer: ``words(max_tokens, max_seqs)`` int32 words in pinned host memory
    and the same words on the device, copied with the rest of the description in the step's
    one host-to-device copy.  ``plan`` fills the host segment from the step's shape and
    returns whatever its parts want to find in ``ctx.plans[name]`` (views of the device
    segment, counts, launch shapes).
    """

    name: str = ""

    def words(self, max_tokens: int, max_seqs: int) -> int:
        return 0

    def plan(self, host, dev: torch.Tensor, q_lens: list[int], starts: list[int]):
        """``q_lens[s]`` tokens of sequence s start at position ``starts[s]``; padding rows of a
        fixed-size batch are included (one token at position 0)."""
        raise NotImplementedError


class Norm(Part):
    """Normalises rows of the 32-bit residual stream.

    ``forward`` returns activations in the compute dtype.  ``add_forward`` first
    adds ``delta`` (a sub-layer's output not yet added) into ``residual`` in
    place, in 32-bit, then normalises; ``rows`` restricts both to some rows and
    leaves ``residual`` untouched (used before the output head).

    A norm whose ``takes_partial_sums`` is True accepts an ``ops.PartialSums`` as ``delta``
    (the float32 slices of a product cut along k, which it adds up itself); the sub-layer
    before it may then hand its output over in that form (``ctx.partial_sums_ok``).
    """

    takes_partial_sums = False

    def forward(self, residual: torch.Tensor, ctx: "StepContext", tag: str = "norm") -> torch.Tensor:
        raise NotImplementedError

    def add_forward(self, residual: torch.Tensor, delta: torch.Tensor | None,
                    ctx: "StepContext", rows: torch.Tensor | None = None,
                    tag: str = "norm") -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    """Puts positions into queries and keys.

    ``encode_and_store`` gets the fused projection output ``qkv``
    ``[tokens, (q_heads + 2 kv_heads) * head_dim]``; it encodes the query heads
    in place, encodes the key heads, and writes keys and values of every token
    to the slot ``ctx.kv_slots[cache.group]`` names (unless ``cache.writes`` is
    False).  One call so that an implementation can fuse both.
    """

    def encode_and_store(self, qkv: torch.Tensor, num_q_heads: int, num_kv_heads: int,
                         head_dim: int, ctx: "StepContext", cache: LayerCache) -> None:
        raise NotImplementedError

    def project_encode_and_store(self, x: torch.Tensor, w_qkv: torch.Tensor, qkv: torch.Tensor,
                                 num_q_heads: int, num_kv_heads: int, head_dim: int,
                                 ctx: "StepContext", cache: LayerCache) -> None:
        """``qkv = x @ w_qkv.T`` followed by ``encode_and_store``.

        An implementation may do both in one kernel; afterwards only the query columns of
        ``qkv`` and the cache are read, so it need not write the key and value columns.
        """
        from .. import ops
        ops.linear(x, w_qkv, qkv)
        self.encode_and_store(qkv, num_q_heads, num_kv_heads, head_dim, ctx, cache)


class Embedding(Part):
    """Token ids -> rows of the float32 residual stream ``[tokens, hidden]``."""

    def forward(self, token_ids: torch.Tensor, ctx: "StepContext") -> torch.Tensor:
        raise NotImplementedError

    def output_matrix(self) -> torch.Tensor:
        """The ``[vocab, hidden]`` matrix a tied output head multiplies by."""
        raise NotImplementedError


class Head(Part):
    """Normalised rows ``[rows, hidden]`` -> float32 logits ``[rows, vocab]``.

    ``bind`` also receives the model's embedding: a tied head takes its matrix from there.
    """

    def bind(self, tensors: dict[str, torch.Tensor], rt: Runtime,
             embedding: "Embedding | None" = None) -> None:
        super().bind(tensors, rt)

    def forward(self, x: torch.Tensor, ctx: "StepContext") -> torch.Tensor:
        raise NotImplementedError


class Mixer(Part):
    """Mixes information across the tokens of a request (attention, or a state)."""

    def cache_spec(self) -> CacheSpec | None:
        return None

    def forward(self, x: torch.Tensor, ctx: "StepContext", cache: LayerCache | None) -> torch.Tensor:
        """``x`` ``[tokens, hidden]`` normalised activations -> output not yet added."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx: "StepContext") -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    """Arrangement of a mixer, a feed-forward and their norms.

    ``forward`` receives the residual stream (float32, updated in place) and
    the previous block's output that is not yet added (``delta``, may be None);
    it returns its own last sub-layer output, again not yet added, so that the
    next norm can fuse the addition.
    """

    mixer: Mixer

    def forward(self, residual: torch.Tensor, delta: torch.Tensor | None,
                ctx: "StepContext", cache: LayerCache | None) -> torch.Tensor:
        raise NotImplementedError

    def first_norm(self) -> "Norm | None":
        """The norm that takes the previous block's pending output (``delta``), if the block
        can tell: the model uses it to learn whether that output may come as partial sums."""
        return None

    def step_planners(self) -> list[type[StepPlanner]]:
        return self.mixer.step_planners()


@dataclass(frozen=True)
class PartSpec:
    """A part chosen by configuration: registry kind plus constructor parameters."""

    kind: str
    params: dict[str, Any] = field(default_factory=dict)

    def __hash__(self) -> int:  # params may hold unhashable values
        return hash(self.kind)
