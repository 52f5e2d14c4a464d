"""Token embedding and output head.

Reference ``ops/embedding.py:49-92``: ``x0[t] = E[id[t]]`` and
``logits = x E^T`` with the head always sharing the embedding matrix
(``model/llama.py:111``).  Here the head shares it only when the configuration
says ``tie_word_embeddings``; otherwise it owns ``lm_head.weight``.  The
residual stream starts in float32, and the logits are written as float32.  Both are
registered kinds (``token_embedding``, ``linear_head``) that a model's plan names, so an
architecture with a scaled embedding or a capped head registers its own.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import Embedding, Head, Runtime, TensorSpec
from .registry import register_embedding, register_head


@register_embedding("token_embedding")
class TokenEmbedding(Embedding):
    def __init__(self, vocab_size: int, hidden_size: int):
        self.vocab_size = int(vocab_size)
        self.hidden_size = int(hidden_size)
        self.weight: torch.Tensor | None = None

    def tensors(self) -> dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.vocab_size, self.hidden_size))}

    def bind(self, tensors, rt: Runtime) -> None:
        super().bind(tensors, rt)
        self.weight = tensors["weight"]

    def forward(self, token_ids: torch.Tensor, ctx) -> torch.Tensor:
        n = token_ids.shape[0]
        residual = ctx.ws.get("residual", (n, self.hidden_size), torch.float32)
        ops.embed_gather(self.weight, token_ids, residual)
        return residual

    def output_matrix(self) -> torch.Tensor:
        return self.weight


@register_head("linear_head")
class OutputHead(Head):
    """``logits = x W^T`` in float32, ``W`` the embedding matrix when tied."""

    def __init__(self, vocab_size: int, hidden_size: int, tied: bool):
        self.vocab_size = int(vocab_size)
        self.hidden_size = int(hidden_size)
        self.tied = bool(tied)
        self.weight: torch.Tensor | None = None

    def tensors(self) -> dict[str, TensorSpec]:
        if self.tied:
            return {}
        return {"weight": TensorSpec((self.vocab_size, self.hidden_size))}

    def bind(self, tensors, rt: Runtime, embedding: Embedding | None = None) -> None:
        super().bind(tensors, rt, embedding)
        self.weight = embedding.output_matrix() if self.tied else tensors["weight"]

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        logits = ctx.ws.get("logits", (x.shape[0], self.vocab_size), torch.float32,
                            row_cap=ctx.ws.max_logit_rows)
        ops.linear(x, self.weight, logits)
        return logits
