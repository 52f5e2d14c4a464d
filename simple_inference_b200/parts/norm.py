"""RMSNorm over the float32 residual stream, with the pending residual add fused in.

Formula (reference ``ops/rmsnorm.py:41-46``): ``y = x * rsqrt(mean(x^2) + eps) * w``
with eps inside the root, no mean subtraction, no bias, the gain multiplying
directly.  The sum of squares, the root and both products are float32; the
result is rounded once to the compute dtype (the reference's Triton form,
``kernels/rmsnorm_kernel.py:105-113``).  The residual adds ``x + h`` of the
reference's block (``model/block.py:138,144``) happen here, in float32, in the
same kernel that reads ``x`` for the norm.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import Norm, Runtime, TensorSpec
from .registry import register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    takes_partial_sums = True   # the kernel adds up the slices of a product cut along k

    def __init__(self, hidden_size: int, eps: float):
        self.hidden_size = int(hidden_size)
        self.eps = float(eps)
        self.weight: torch.Tensor | None = None

    def tensors(self) -> dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.hidden_size,), kind="vector", init="gain")}

    def bind(self, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        super().bind(tensors, rt)
        self.weight = tensors["weight"]

    def forward(self, residual, ctx, tag: str = "norm"):
        return self.add_forward(residual, None, ctx, None, tag)

    def add_forward(self, residual, delta, ctx, rows=None, tag: str = "norm"):
        n = residual.shape[0] if rows is None else rows.shape[0]
        out = ctx.ws.get(tag + ".out", (n, self.hidden_size), self.rt.dtype)
        ops.rmsnorm(residual, self.weight, self.eps, out, delta=delta, rows=rows)
        return out
