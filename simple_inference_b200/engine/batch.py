"""The flat batch of one step and its device-side description.

A step gets a list of ``StepEntry``: for each request its next tokens (a
portion of its prompt, or one decoded token) and the places among them whose
logits are wanted.  All entries run as one batch of ``N`` tokens in ``S``
sequences.  ``BatchBuilder`` lays the integers the kernels need into ONE pinned
host buffer with a fixed layout and copies it to ONE device buffer per step;
``StepContext`` holds views of that buffer:

    token_ids[N] positions[N] tok_seq[N]      per token
    kv_slots[g][N]                            per token and layer group: page*page_size+offset
    cu_q[S+1] seq_slots[S]                    per sequence: token range, state slot
    block_tables[g][S, max_pages_g]           per sequence and layer group
    logit_rows[R]                             token indices whose logits are wanted
    single_seqs[...] tile_seq[...] tile_start[...]   routing for the attention kernels:
        sequences with exactly one token, and 64-token query tiles of the others

The layout is fixed by the capacities, so the same device addresses serve every
step and every captured graph.  The reference rebuilds an int64 ``(B,
max_blocks)`` table from Python lists and copies ids, positions and cos/sin
rows separately each step (``serving/paged_decoder.py:207-257``).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable

import numpy as np
import torch

from ..cache.manager import CacheManager, pages_for

QUERY_TILE = 64  # query rows per block of the mma.sync prefill kernel
WIDE_TILE = 128  # query rows per block of the tcgen05 prefill kernel


@dataclass
class StepEntry:
    request: Hashable
    tokens: list[int]
    want: list[int] = field(default_factory=list)  # indices into ``tokens``


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


class Workspace:
    """Named scratch buffers with stable addresses.

    A buffer is allocated once, for ``row_cap`` rows of the width first asked
    for (default cap: the most tokens a step may hold), and never moves
    afterwards, so a captured graph can keep its address.  Asking for more
    than the capacity after ``freeze()`` is an error rather than a silent move.
    """

    def __init__(self, device: torch.device, max_rows: int, max_logit_rows: int | None = None):
        self.device = device
        self.max_rows = max_rows
        self.max_logit_rows = max_logit_rows if max_logit_rows is not None else max_rows
        self._buffers: dict[tuple[str, torch.dtype], torch.Tensor] = {}
        self._frozen = False

    def freeze(self) -> None:
        self._frozen = True

    def get(self, tag: str, shape: tuple[int, ...], dtype: torch.dtype,
            row_cap: int | None = None) -> torch.Tensor:
        width = 1
        for s in shape[1:]:
            width *= s
        numel = shape[0] * width
        key = (tag, dtype)
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < numel:
            if self._frozen and buf is not None:
                raise RuntimeError(f"workspace buffer {tag!r} would move after a graph was "
                                   f"captured (asked for {shape})")
            cap = max(shape[0], row_cap if row_cap is not None else self.max_rows)
            buf = torch.empty(max(cap * width, 1), dtype=dtype, device=self.device)
            self._buffers[key] = buf
        return buf[:numel].view(shape)


@dataclass
class StepContext:
    n_tokens: int
    n_seqs: int
    num_logit_rows: int
    token_ids: torch.Tensor
    positions: torch.Tensor
    tok_seq: torch.Tensor
    kv_slots: list[torch.Tensor]
    cu_q: torch.Tensor
    seq_slots: torch.Tensor
    block_tables: list[torch.Tensor]
    logit_rows: torch.Tensor
    single_seqs: torch.Tensor
    n_single: int
    tile_seq: torch.Tensor
    tile_start: torch.Tensor
    n_tiles: int
    tile_pairs: torch.Tensor
    n_pairs: int
    wide_seq: torch.Tensor    # the same portions cut into WIDE_TILE-query tiles, longest first
    wide_start: torch.Tensor
    n_wide: int
    max_kv_len: int
    max_q_len: int
    max_seqs: int
    ws: Workspace
    # host copies for parts that plan on the host
    q_lens: list[int] = field(default_factory=list)
    kv_lens: list[int] = field(default_factory=list)
    fixed_shape: bool = False  # True inside a captured decode graph (sizes are capacities)


class BatchBuilder:
    def __init__(self, cache: CacheManager, max_tokens: int, max_seqs: int, max_seq_len: int,
                 device: torch.device):
        self.cache = cache
        self.device = device
        self.max_tokens = max_tokens
        self.max_seqs = max_seqs
        self.max_seq_len = max_seq_len
        self.n_groups = len(cache.groups)
        self.table_len = [pages_for(max_seq_len, g.page_size) for g in cache.groups]
        self.max_tiles = (max_tokens // QUERY_TILE + max_seqs + 2) // 2 * 2

        off = 0
        self._off: dict[str, tuple[int, int]] = {}

        def seg(name: str, n: int) -> None:
            nonlocal off
            self._off[name] = (off, n)
            off += (n + 3) // 4 * 4  # keep every segment 16-byte aligned

        seg("cu_q", max_seqs + 1)
        seg("seq_slots", max_seqs)
        seg("single_seqs", max_seqs)
        seg("tile_seq", self.max_tiles)
        seg("tile_start", self.max_tiles)
        seg("tile_pairs", self.max_tiles + 1)
        seg("wide_seq", self.max_tiles)
        seg("wide_start", self.max_tiles)
        for g in range(self.n_groups):
            seg(f"block_table{g}", max_seqs * self.table_len[g])
        seg("token_ids", max_tokens)
        seg("positions", max_tokens)
        seg("tok_seq", max_tokens)
        seg("logit_rows", max_tokens)
        for g in range(self.n_groups):
            seg(f"kv_slots{g}", max_tokens)
        self.total = off
        pin = device.type == "cuda"
        self.host = torch.zeros(self.total, dtype=torch.int32, pin_memory=pin)
        self.host_np = self.host.numpy()
        self.dev = torch.zeros(self.total, dtype=torch.int32, device=device)
        self._copied = torch.cuda.Event() if pin else None
        self._copy_pending = False
        # what each block-table row of the host buffer holds: (admission serial, entries written),
        # so that a request that keeps its row from step to step only appends its new pages
        self._row_owner: list[list[tuple[int, int] | None]] = [
            [None] * max_seqs for _ in range(self.n_groups)]
        # views of the two buffers are made once per distinct set of sizes: slicing a torch
        # tensor costs more than filling a decode step's numbers
        self._host_views: dict[str, np.ndarray] = {}
        self._device_views: dict[tuple, dict] = {}

    def _h(self, name: str) -> np.ndarray:
        v = self._host_views.get(name)
        if v is None:
            o, n = self._off[name]
            v = self._host_views[name] = self.host_np[o:o + n]
        return v

    def _d(self, name: str, n: int | None = None) -> torch.Tensor:
        o, cap = self._off[name]
        return self.dev[o:o + (cap if n is None else n)]

    def build(self, entries: list[StepEntry], starts: list[int], ws: Workspace,
              pad_to: int | None = None) -> StepContext:
        """Fill the buffers for ``entries`` (``starts[i]`` = position of entry i's first token).

        ``pad_to``: make a decode-only batch of exactly that many sequences by
        adding rows that read and write only the scratch page and scratch slot.
        """
        if self._copy_pending:
            self._copied.synchronize()
            self._copy_pending = False
        cache = self.cache
        S = len(entries)
        N = sum(len(e.tokens) for e in entries)
        pad = 0 if pad_to is None else pad_to - S
        if pad < 0 or (pad_to is not None and any(len(e.tokens) != 1 for e in entries)):
            raise ValueError("padding is for decode-only batches no larger than the bucket")
        if S + pad > self.max_seqs or N + pad > self.max_tokens:
            raise ValueError(f"step of {N} tokens in {S} sequences exceeds the capacities "
                             f"({self.max_tokens} tokens, {self.max_seqs} sequences)")

        cu_q = self._h("cu_q"); seq_slots = self._h("seq_slots")
        token_ids = self._h("token_ids"); positions = self._h("positions")
        tok_seq = self._h("tok_seq"); logit_rows = self._h("logit_rows")
        single = self._h("single_seqs"); tile_seq = self._h("tile_seq")
        tile_start = self._h("tile_start")
        tile_pairs = self._h("tile_pairs")
        tile_work: list[int] = []
        wide: list[tuple[int, int, int]] = []  # (keys its last row sees, sequence, first row)
        tables = [self._h(f"block_table{g}").reshape(self.max_seqs, self.table_len[g])
                  for g in range(self.n_groups)]
        kv_slots = [self._h(f"kv_slots{g}") for g in range(self.n_groups)]

        t = 0; r = 0; n_single = 0; n_tiles = 0
        q_lens: list[int] = []; kv_lens: list[int] = []
        cu_q[0] = 0
        for s, (e, start) in enumerate(zip(entries, starts)):
            n = len(e.tokens)
            end = start + n
            if end > self.max_seq_len:
                raise ValueError(f"request {e.request!r} would reach {end} tokens, beyond "
                                 f"max_seq_len {self.max_seq_len}")
            seq_slots[s] = cache.slot(e.request)
            if n == 1:
                token_ids[t] = e.tokens[0]
                positions[t] = start
                tok_seq[t] = s
            else:
                token_ids[t:t + n] = e.tokens
                positions[t:t + n] = np.arange(start, end, dtype=np.int32)
                tok_seq[t:t + n] = s
            for g, grp in enumerate(cache.groups):
                table = cache.block_table(e.request, g)
                row = tables[g][s]
                owner = self._row_owner[g][s]
                serial = cache.admission(e.request)
                if grp.spec.window is None and owner is not None and owner[0] == serial \
                        and owner[1] <= len(table):
                    if owner[1] < len(table):
                        row[owner[1]:len(table)] = table[owner[1]:]   # only the new pages
                else:
                    row[:len(table)] = table
                self._row_owner[g][s] = (serial, len(table))
                ps = grp.page_size
                if n == 1:
                    page = table[start // ps]
                    if page < 0:
                        raise RuntimeError(f"request {e.request!r} writes to a page already given back")
                    kv_slots[g][t] = page * ps + start % ps
                else:
                    where = np.arange(start, end)
                    pages = np.asarray(table, dtype=np.int64)[where // ps]
                    if (pages < 0).any():
                        raise RuntimeError(f"request {e.request!r} writes to a page already given back")
                    kv_slots[g][t:t + n] = pages * ps + where % ps
            for w in e.want:
                if not (0 <= w < n):
                    raise ValueError(f"want index {w} outside the {n} tokens of {e.request!r}")
                logit_rows[r] = t + w
                r += 1
            if n == 1:
                single[n_single] = s
                n_single += 1
            else:
                for q0 in range(0, n, QUERY_TILE):
                    tile_seq[n_tiles] = s
                    tile_start[n_tiles] = q0
                    tile_work.append(start + min(q0 + QUERY_TILE, n))  # keys its last row sees
                    n_tiles += 1
                for q0 in range(0, n, WIDE_TILE):
                    wide.append((start + min(q0 + WIDE_TILE, n), s, q0))
            q_lens.append(n); kv_lens.append(end)
            t += n
            cu_q[s + 1] = t
        for k in range(pad):  # padding rows: one token at position 0 on the scratch page
            s = S + k
            token_ids[t] = 0; positions[t] = 0; tok_seq[t] = s
            seq_slots[s] = cache.scratch_slot
            for g, grp in enumerate(cache.groups):
                tables[g][s, 0] = grp.scratch_page
                self._row_owner[g][s] = None
                kv_slots[g][t] = grp.scratch_page * grp.page_size
            single[n_single] = s; n_single += 1
            logit_rows[r] = t; r += 1
            q_lens.append(1); kv_lens.append(1)
            t += 1
            cu_q[s + 1] = t
        S += pad; N = t
        n_pairs = pair_tiles(tile_work, tile_pairs)
        if wide:
            wide.sort(key=lambda w: -w[0])
            ws_, wq_ = self._h("wide_seq"), self._h("wide_start")
            for i, (_, s, q0) in enumerate(wide):
                ws_[i] = s
                wq_[i] = q0

        self.dev.copy_(self.host, non_blocking=True)
        if self._copied is not None:
            self._copied.record()
            self._copy_pending = True

        sizes = (N, S, r, n_single, n_tiles, n_pairs, len(wide))
        views = self._device_views.get(sizes)
        if views is None:
            if len(self._device_views) >= 512:
                self._device_views.clear()
            views = self._device_views[sizes] = dict(
                token_ids=self._d("token_ids", N), positions=self._d("positions", N),
                tok_seq=self._d("tok_seq", N),
                kv_slots=[self._d(f"kv_slots{g}", N) for g in range(self.n_groups)],
                cu_q=self._d("cu_q", S + 1), seq_slots=self._d("seq_slots", S),
                block_tables=[self._d(f"block_table{g}").view(self.max_seqs, self.table_len[g])[:S]
                              for g in range(self.n_groups)],
                logit_rows=self._d("logit_rows", r),
                single_seqs=self._d("single_seqs", n_single),
                tile_seq=self._d("tile_seq", n_tiles), tile_start=self._d("tile_start", n_tiles),
                tile_pairs=self._d("tile_pairs", 2 * n_pairs),
                wide_seq=self._d("wide_seq", len(wide)), wide_start=self._d("wide_start", len(wide)))
        return StepContext(
            n_tokens=N, n_seqs=S, num_logit_rows=r, n_single=n_single, n_tiles=n_tiles,
            n_pairs=n_pairs, n_wide=len(wide), max_kv_len=max(kv_lens) if kv_lens else 0,
            max_q_len=max(q_lens) if q_lens else 0, max_seqs=self.max_seqs, ws=ws, q_lens=q_lens,
            kv_lens=kv_lens, **views,
        )
