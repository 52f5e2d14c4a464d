"""Rotary position encoding with the llama3 frequency scaling.

Frequencies (reference ``ops/rope.py:97-98``): ``inv_freq_i = theta^(-2i/D)``
for ``i < D/2``, computed in float32.  With ``rope_type == "llama3"`` each
frequency f is rescaled by its wavelength ``wl = 2*pi/f``
(reference ``ops/rope.py:136-155``):

    wl < orig/high_freq_factor          -> f
    wl > orig/low_freq_factor           -> f / factor
    otherwise, s = (orig/wl - low) / (high - low) -> (1-s) * f/factor + s * f

in double precision per frequency, stored as float32.  Any other ``rope_type``
leaves the frequencies alone (``ops/rope.py:101``).  The rotation itself (split
halves, pairs ``(x_i, x_{i+D/2})``, reference ``ops/rope.py:167-215``) runs in
the kernel that also writes keys and values to their pages; it forms
``angle = float(position) * inv_freq_i`` in float32 as the reference's table
does (``ops/rope.py:108-110``) and keeps cos, sin and the products in float32.
"""

from __future__ import annotations

import math

import torch

from .. import ops
from .base import LayerCache, PositionEncoding, Runtime
from .registry import register_position_encoding


def rope_inverse_frequencies(head_dim: int, theta: float, scaling: dict | None) -> torch.Tensor:
    """float32 ``[head_dim/2]`` rotation frequencies, scaled if ``scaling`` says llama3."""
    exponents = torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim
    inv_freq = 1.0 / (torch.tensor(float(theta), dtype=torch.float32) ** exponents)
    if scaling is None or scaling.get("rope_type", "default") != "llama3":
        return inv_freq
    factor = float(scaling["factor"])
    low, high = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
    orig = float(scaling["original_max_position_embeddings"])
    longest, shortest = orig / low, orig / high  # wavelength bounds of the blend band
    scaled = []
    for f in inv_freq.tolist():
        wavelength = 2.0 * math.pi / f
        if wavelength < shortest:
            scaled.append(f)
        elif wavelength > longest:
            scaled.append(f / factor)
        else:
            blend = (orig / wavelength - low) / (high - low)
            scaled.append((1.0 - blend) * f / factor + blend * f)
    return torch.tensor(scaled, dtype=torch.float32)


@register_position_encoding("rope")
class RotaryEmbedding(PositionEncoding):
    def __init__(self, head_dim: int, theta: float, scaling: dict | None = None):
        self.head_dim = int(head_dim)
        self.theta = float(theta)
        self.scaling = dict(scaling) if scaling else None
        self.inv_freq: torch.Tensor | None = None

    def bind(self, tensors, rt: Runtime) -> None:
        super().bind(tensors, rt)
        self.inv_freq = rope_inverse_frequencies(self.head_dim, self.theta, self.scaling).to(rt.device)

    def encode_and_store(self, qkv, num_q_heads, num_kv_heads, head_dim, ctx, cache: LayerCache):
        ops.rope_kv_store(qkv, ctx.positions, self.inv_freq, ctx.kv_slots[cache.group], cache.pool,
                          num_q_heads, num_kv_heads, head_dim, cache.page_size, cache.writes)

    def project_encode_and_store(self, x, w_qkv, qkv, num_q_heads, num_kv_heads, head_dim, ctx,
                                 cache: LayerCache):
        # a few tokens (decoding): the rotation and the cache write are the projection's epilogue
        if ops.can_fuse_projection_rope(x, w_qkv, qkv):
            ops.linear_rope_kv_store(x, w_qkv, qkv, ctx.positions, self.inv_freq,
                                     ctx.kv_slots[cache.group], cache.pool, num_q_heads,
                                     num_kv_heads, head_dim, cache.page_size, cache.writes)
        else:
            super().project_encode_and_store(x, w_qkv, qkv, num_q_heads, num_kv_heads, head_dim,
                                             ctx, cache)


@register_position_encoding("none")
class NoPositionEncoding(PositionEncoding):
    """No encoding: keys and values are stored as projected (rotation by angle 0)."""

    def __init__(self, head_dim: int):
        self.head_dim = int(head_dim)
        self.inv_freq: torch.Tensor | None = None

    def bind(self, tensors, rt: Runtime) -> None:
        super().bind(tensors, rt)
        self.inv_freq = torch.zeros(self.head_dim // 2, dtype=torch.float32, device=rt.device)

    def encode_and_store(self, qkv, num_q_heads, num_kv_heads, head_dim, ctx, cache: LayerCache):
        ops.rope_kv_store(qkv, ctx.positions, self.inv_freq, ctx.kv_slots[cache.group], cache.pool,
                          num_q_heads, num_kv_heads, head_dim, cache.page_size, cache.writes)

    def project_encode_and_store(self, x, w_qkv, qkv, num_q_heads, num_kv_heads, head_dim, ctx,
                                 cache: LayerCache):
        # a few tokens (decoding): the rotation and the cache write are the projection's epilogue
        if ops.can_fuse_projection_rope(x, w_qkv, qkv):
            ops.linear_rope_kv_store(x, w_qkv, qkv, ctx.positions, self.inv_freq,
                                     ctx.kv_slots[cache.group], cache.pool, num_q_heads,
                                     num_kv_heads, head_dim, cache.page_size, cache.writes)
        else:
            super().project_encode_and_store(x, w_qkv, qkv, num_q_heads, num_kv_heads, head_dim,
                                             ctx, cache)
