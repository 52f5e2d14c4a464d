"""Grouped-query attention over the paged cache.

Reference ``ops/attention.py:70-228``: ``q = x Wq^T``, ``k = x Wk^T``,
``v = x Wv^T`` without bias (``:128-130``), heads of ``head_dim`` columns
(``:133-135``), position encoding on q and k before the cache write (``:146``),
query head h reads key/value head ``h // groups``
(``kernels/attention_kernel.py:188``), scores scaled by ``1/sqrt(head_dim)``
(``:289-290``), causal mask by absolute position, softmax in float32, then
``out = merge_heads(O) Wo^T`` (``:223-226``).  Here the three projections are
one product with ``[Wq; Wk; Wv]`` stacked by rows, and the keys and values of
the step's tokens are written to their pages before attention reads the pages,
so a portion of a prompt attends to itself through the cache.

``window`` (None for Llama) limits each query to the last ``window`` keys; the
cache then gives pages back as the window passes them.
"""

from __future__ import annotations

import math

import torch

from .. import ops
from .attention_plan import PagedAttentionPlanner
from .base import LayerCache, Mixer, PagedKVSpec, PartSpec, Runtime, StepPlanner, TensorSpec
from .registry import POSITION_ENCODINGS, register_mixer


@register_mixer("attention")
class PagedAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position: PartSpec, window: int | None = None, scale: float | None = None):
        if num_heads % num_kv_heads != 0:
            raise ValueError(f"{num_heads} query heads do not divide into {num_kv_heads} groups")
        if head_dim % 16 != 0 or not (16 <= head_dim <= 256):
            raise ValueError(f"head_dim {head_dim}: the attention kernels take multiples of 16 "
                             f"from 16 to 256")
        self.hidden_size = int(hidden_size)
        self.num_heads = int(num_heads)
        self.num_kv_heads = int(num_kv_heads)
        self.head_dim = int(head_dim)
        self.window = int(window) if window else None
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.position = POSITION_ENCODINGS.build(position)
        self.q_width = self.num_heads * self.head_dim
        self.kv_width = self.num_kv_heads * self.head_dim
        self.w_qkv: torch.Tensor | None = None
        self.w_o: torch.Tensor | None = None

    def tensors(self) -> dict[str, TensorSpec]:
        return {
            "wq": TensorSpec((self.q_width, self.hidden_size)),
            "wk": TensorSpec((self.kv_width, self.hidden_size)),
            "wv": TensorSpec((self.kv_width, self.hidden_size)),
            "wo": TensorSpec((self.hidden_size, self.q_width)),
        }

    def cache_spec(self) -> PagedKVSpec:
        return PagedKVSpec(self.num_kv_heads, self.head_dim, self.window)

    def step_planners(self) -> list[type[StepPlanner]]:
        return [PagedAttentionPlanner]  # which kernel each sequence of the step goes to

    def bind(self, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        super().bind(tensors, rt)
        self.w_qkv = torch.cat([tensors["wq"], tensors["wk"], tensors["wv"]], dim=0).contiguous()
        self.w_o = tensors["wo"]
        self.position.bind({}, rt)

    def forward(self, x: torch.Tensor, ctx, cache: LayerCache) -> torch.Tensor:
        n = x.shape[0]
        qkv = ctx.ws.get("attn.qkv", (n, self.q_width + 2 * self.kv_width), x.dtype)
        self.position.project_encode_and_store(x, self.w_qkv, qkv, self.num_heads,
                                               self.num_kv_heads, self.head_dim, ctx, cache)
        mixed = ctx.ws.get("attn.mixed", (n, self.q_width), x.dtype)
        ops.paged_attention(qkv, cache.pool, ctx, ctx.plans.get(PagedAttentionPlanner.name),
                            cache.group, mixed, self.num_heads,
                            self.num_kv_heads, self.head_dim, self.scale, self.window)
        return ops.linear_for_residual(mixed, self.w_o, ctx.ws, "attn.proj",
                                       getattr(ctx, "partial_sums_ok", False))
