"""What the paged-attention kernels want to know about a step, worked out once per step.

The bfloat16 attention kernels are three: one for sequences that bring a single
token (decoding), one that works on 64-query tiles (``mma.sync``) and one that
works on 128-query tiles (tcgen05).  Which sequence goes where, the tiles of the
longer portions, and the pairing of long with short tiles depend only on the
step's shape, not on the layer, so every attention layer of a model shares one
``AttentionStepPlan`` made by ``PagedAttentionPlanner``.  The planner's lists live
in a segment of the step's description buffer and reach the device in the step's
one copy.

Nothing outside the attention mixer knows these lists: a mixer with kernels of
another geometry brings a planner of its own.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from .base import StepPlanner

QUERY_TILE = 64   # query rows per block of the mma.sync prefill kernel
WIDE_TILE = 128   # query rows per block of the tcgen05 prefill kernel


def pair_tiles(work: list[int], out) -> int:
    """Pair query tiles for the prefill attention kernel: longest with shortest.

    ``work[i]`` is the number of keys tile i attends to.  Writes pairs of tile
    indices into ``out`` (second index -1 for an odd one out) and returns the
    number of pairs.  A block runs the two tiles of a pair back to back, so every
    block of a causal prompt does about the same amount of work.
    """
    order = sorted(range(len(work)), key=lambda i: -work[i])
    n_pairs = (len(order) + 1) // 2
    for k in range(n_pairs):
        a, b = order[k], (order[len(order) - 1 - k] if len(order) - 1 - k > k else -1)
        out[2 * k] = a
        out[2 * k + 1] = b
    return n_pairs


@dataclass
class AttentionStepPlan:
    single_seqs: torch.Tensor   # sequences with exactly one token
    n_single: int
    tile_seq: torch.Tensor      # the other sequences cut into QUERY_TILE-query tiles
    tile_start: torch.Tensor
    n_tiles: int
    tile_pairs: torch.Tensor    # tiles paired long with short
    n_pairs: int
    wide_seq: torch.Tensor      # the same portions cut into WIDE_TILE-query tiles, longest first
    wide_start: torch.Tensor
    n_wide: int
    max_q_len: int


class PagedAttentionPlanner(StepPlanner):
    name = "paged_attention"

    def __init__(self):
        self._seg: dict[str, tuple[int, int]] = {}
        self._views: dict[tuple, dict] = {}
        self._dev: torch.Tensor | None = None
        self._host: np.ndarray | None = None
        self._h: dict[str, np.ndarray] = {}
        self._all_single = -1   # how many leading entries of single_seqs hold 0, 1, 2, ... already

    def words(self, max_tokens: int, max_seqs: int) -> int:
        max_tiles = (max_tokens // QUERY_TILE + max_seqs + 2) // 2 * 2
        off = 0
        for name, n in (("single_seqs", max_seqs), ("tile_seq", max_tiles),
                        ("tile_start", max_tiles), ("tile_pairs", max_tiles + 1),
                        ("wide_seq", max_tiles), ("wide_start", max_tiles)):
            self._seg[name] = (off, n)
            off += (n + 3) // 4 * 4   # every list starts on a 16-byte boundary
        return off

    def plan(self, host: np.ndarray, dev: torch.Tensor, q_lens: list[int],
             starts: list[int]) -> AttentionStepPlan:
        if self._host is not host:
            self._host, self._all_single = host, -1
            self._h = {name: host[o:o + n] for name, (o, n) in self._seg.items()}
        h = self._h
        if max(q_lens) == 1:   # decoding only: every sequence is single, and the list is 0, 1, 2, ...
            n = len(q_lens)
            if self._all_single < n:
                h["single_seqs"][:n] = np.arange(n, dtype=np.int32)
                self._all_single = n
            return self._result(dev, n, 0, 0, 0, 1)
        self._all_single = -1
        n_single = n_tiles = 0
        tile_work: list[int] = []
        wide: list[tuple[int, int, int]] = []  # (keys its last row sees, sequence, first row)
        for s, (n, start) in enumerate(zip(q_lens, starts)):
            if n == 1:
                h["single_seqs"][n_single] = s
                n_single += 1
                continue
            for q0 in range(0, n, QUERY_TILE):
                h["tile_seq"][n_tiles] = s
                h["tile_start"][n_tiles] = q0
                tile_work.append(start + min(q0 + QUERY_TILE, n))  # keys its last row sees
                n_tiles += 1
            for q0 in range(0, n, WIDE_TILE):
                wide.append((start + min(q0 + WIDE_TILE, n), s, q0))
        n_pairs = pair_tiles(tile_work, h["tile_pairs"])
        wide.sort(key=lambda w: -w[0])
        for i, (_, s, q0) in enumerate(wide):
            h["wide_seq"][i] = s
            h["wide_start"][i] = q0

        return self._result(dev, n_single, n_tiles, n_pairs, len(wide), max(q_lens) if q_lens else 0)

    def _result(self, dev: torch.Tensor, n_single: int, n_tiles: int, n_pairs: int, n_wide: int,
                max_q_len: int) -> AttentionStepPlan:
        if self._dev is not dev:
            self._dev, self._views = dev, {}
        sizes = (n_single, n_tiles, n_pairs, n_wide)
        v = self._views.get(sizes)
        if v is None:  # views are made once per distinct set of sizes: slicing costs more than filling
            if len(self._views) >= 512:
                self._views.clear()

            def d(name: str, n: int) -> torch.Tensor:
                o, _ = self._seg[name]
                return dev[o:o + n]
            v = self._views[sizes] = dict(
                single_seqs=d("single_seqs", n_single), tile_seq=d("tile_seq", n_tiles),
                tile_start=d("tile_start", n_tiles), tile_pairs=d("tile_pairs", 2 * n_pairs),
                wide_seq=d("wide_seq", n_wide), wide_start=d("wide_start", n_wide))
        return AttentionStepPlan(n_single=n_single, n_tiles=n_tiles, n_pairs=n_pairs,
                                 n_wide=n_wide, max_q_len=max_q_len, **v)


def plan_on_device(q_lens: list[int], starts: list[int], device: torch.device) -> AttentionStepPlan:
    """A plan in buffers of its own (for callers outside the step function, such as kernel tests)."""
    planner = PagedAttentionPlanner()
    words = planner.words(sum(q_lens), len(q_lens))
    host = np.zeros(words, dtype=np.int32)
    dev = torch.zeros(words, dtype=torch.int32, device=device)
    plan = planner.plan(host, dev, q_lens, starts)
    dev.copy_(torch.from_numpy(host))
    return plan
