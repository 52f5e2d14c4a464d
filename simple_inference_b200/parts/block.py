"""Arrangements of a mixer, a feed-forward and their norms.

``prenorm`` is the reference's block (``model/block.py:119-146``):
``h = x + Mixer(Norm_a(x)); out = h + FeedForward(Norm_b(h))``.  The residual
stream ``x`` is float32 and updated in place; each addition is done by the norm
that follows it, so a block hands its last sub-layer output on without adding it.
"""

from __future__ import annotations

import torch

from .base import Block, LayerCache, PartSpec, Runtime, TensorSpec
from .registry import FEED_FORWARDS, MIXERS, NORMS, register_block


@register_block("prenorm")
class PreNormBlock(Block):
    def __init__(self, mixer: PartSpec, mixer_norm: PartSpec, feed_forward: PartSpec,
                 feed_forward_norm: PartSpec):
        self.mixer_norm = NORMS.build(mixer_norm)
        self.mixer = MIXERS.build(mixer)
        self.feed_forward_norm = NORMS.build(feed_forward_norm)
        self.feed_forward = FEED_FORWARDS.build(feed_forward)

    def _children(self):
        return (("mixer_norm", self.mixer_norm), ("mixer", self.mixer),
                ("feed_forward_norm", self.feed_forward_norm), ("feed_forward", self.feed_forward))

    def tensors(self) -> dict[str, TensorSpec]:
        out: dict[str, TensorSpec] = {}
        for prefix, part in self._children():
            for name, spec in part.tensors().items():
                out[f"{prefix}.{name}"] = spec
        return out

    def bind(self, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        super().bind(tensors, rt)
        for prefix, part in self._children():
            own = {k[len(prefix) + 1:]: v for k, v in tensors.items() if k.startswith(prefix + ".")}
            part.bind(own, rt)

    def first_norm(self):
        return self.mixer_norm

    def forward(self, residual, delta, ctx, cache: LayerCache | None):
        # ctx.partial_sums_ok tells a sub-layer whether the norm that will add its output takes
        # partial sums: for the mixer that is this block's second norm, for the feed-forward
        # whatever follows the block (the model said so in ctx.next_takes_partial_sums)
        after_block = getattr(ctx, "next_takes_partial_sums", False)
        h = self.mixer_norm.add_forward(residual, delta, ctx)
        ctx.partial_sums_ok = self.feed_forward_norm.takes_partial_sums
        mixed = self.mixer.forward(h, ctx, cache)
        h = self.feed_forward_norm.add_forward(residual, mixed, ctx)
        ctx.partial_sums_ok = after_block
        out = self.feed_forward.forward(h, ctx)
        ctx.partial_sums_ok = False
        return out
