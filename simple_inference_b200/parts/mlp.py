"""SwiGLU feed-forward.

Reference ``ops/mlp.py:61-128``: ``[g | u] = x W_gu^T`` with
``W_gu = cat([W_gate, W_up], dim=0)`` (``:87,104,117-118``),
``h = silu(g) * u`` (``:125``; float32 arithmetic as in
``kernels/swiglu_kernel.py:142-150``), ``y = h W_down^T`` (``:128``).  Dense:
every token goes through the same two matrices.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, Runtime, TensorSpec
from .registry import register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.w_gate_up: torch.Tensor | None = None
        self.w_down: torch.Tensor | None = None

    def tensors(self) -> dict[str, TensorSpec]:
        return {
            "w_gate": TensorSpec((self.intermediate_size, self.hidden_size)),
            "w_up": TensorSpec((self.intermediate_size, self.hidden_size)),
            "w_down": TensorSpec((self.hidden_size, self.intermediate_size)),
        }

    def bind(self, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        super().bind(tensors, rt)
        self.w_gate_up = torch.cat([tensors["w_gate"], tensors["w_up"]], dim=0).contiguous()
        self.w_down = tensors["w_down"]

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        n = x.shape[0]
        hidden = ctx.ws.get("mlp.hidden", (n, self.intermediate_size), x.dtype)
        if ops.can_fuse_swiglu(x, self.w_gate_up):
            # a few tokens: one weight-streaming kernel with the gate fused in
            ops.linear_swiglu(x, self.w_gate_up, hidden)
        else:
            gate_up = ctx.ws.get("mlp.gate_up", (n, 2 * self.intermediate_size), x.dtype)
            ops.linear(x, self.w_gate_up, gate_up)
            ops.swiglu(gate_up, hidden)
        return ops.linear_for_residual(hidden, self.w_down, ctx.ws, "mlp.down",
                                       getattr(ctx, "partial_sums_ok", False))
