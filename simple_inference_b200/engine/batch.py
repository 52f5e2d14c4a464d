"""The flat batch of one step and its device-side description.

A step gets a list of ``StepEntry``: for each request its next tokens (a
portion of its prompt, or one decoded token) and the places among them whose
logits are wanted.  All entries run as one batch of ``N`` tokens in ``S``
sequences.  ``BatchBuilder`` lays the integers the kernels need into ONE pinned
host buffer with a fixed layout, mirrored by ONE device buffer; ``StepContext``
holds views of the device buffer:

    cu_q[S+1] seq_slots[S]                    per sequence: token range, state slot
    token_ids[N] positions[N] tok_seq[N]      per token
    logit_rows[R]                             token indices whose logits are wanted
    kv_slots[g][N]                            per token and layer group: page*page_size+offset
    (a segment for every step planner of the model's parts, see parts/base.py)
    block_tables[g][S, max_pages_g]           per sequence and layer group

Everything but the block tables reaches the device in one copy per step; of the
block tables only what changed since the last step is copied (the pages a request
gained, or the rows of requests that moved), so a step's copy does not grow with the
longest sequence the engine allows.  The layout is fixed by the capacities, so the
same device addresses serve every step and every captured graph.  The reference
rebuilds an int64 ``(B, max_blocks)`` table from Python lists and copies ids,
positions and cos/sin rows separately each step (``serving/paged_decoder.py:207-257``).

What a particular kind of mixer wants planned per step (the attention kernels'
routing lists, for one) is not known here: the model's parts name ``StepPlanner``
classes, each gets a segment of the buffer, and its result is found in
``ctx.plans[name]``.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Hashable

import numpy as np
import torch

from ..cache.manager import CacheManager, pages_for
from ..parts.base import StepPlanner


@dataclass
class StepEntry:
    request: Hashable
    tokens: list[int]
    want: list[int] = field(default_factory=list)  # indices into ``tokens``


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
        self._views: dict[tuple, torch.Tensor] = {}
        self._frozen = False

    def freeze(self) -> None:
        self._frozen = True

    def get(self, tag: str, shape: tuple[int, ...], dtype: torch.dtype,
            row_cap: int | None = None) -> torch.Tensor:
        vkey = (tag, dtype, shape)
        view = self._views.get(vkey)
        if view is not None:   # the same buffer cut the same way as before: no arithmetic, no new view
            return view
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
            for k in [k for k in self._views if k[0] == tag and k[1] == dtype]:
                del self._views[k]   # views of the buffer this one replaces
        if len(self._views) >= 4096:
            self._views.clear()
        view = self._views[vkey] = buf[:numel].view(shape)
        return view


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
    max_kv_len: int
    max_q_len: int
    max_seqs: int
    ws: Workspace
    # host copies for parts that plan on the host
    q_lens: list[int] = field(default_factory=list)
    kv_lens: list[int] = field(default_factory=list)
    plans: dict[str, Any] = field(default_factory=dict)  # what each step planner returned
    fixed_shape: bool = False  # True inside a captured decode graph (sizes are capacities)
    # set by the model and the blocks as the step runs: whether the norm that will add the
    # output of the sub-layer now running takes ops.PartialSums (parts/base.py, Norm)
    partial_sums_ok: bool = False
    next_takes_partial_sums: bool = False


_FEW_ROWS = 8            # up to this many changed block-table rows are copied span by span,
_ONE_COPY_WORDS = 1 << 16  # more of them as one block of whole rows if that stays this small


class BatchBuilder:
    def __init__(self, cache: CacheManager, max_tokens: int, max_seqs: int, max_seq_len: int,
                 device: torch.device, planners: dict[str, type[StepPlanner]] | None = None):
        self.cache = cache
        self.device = device
        self.max_tokens = max_tokens
        self.max_seqs = max_seqs
        self.max_seq_len = max_seq_len
        self.n_groups = len(cache.groups)
        self.table_len = [pages_for(max_seq_len, g.page_size) for g in cache.groups]
        self.planners: dict[str, StepPlanner] = {name: cls() for name, cls in (planners or {}).items()}

        off = 0
        self._off: dict[str, tuple[int, int]] = {}

        def seg(name: str, n: int) -> None:
            nonlocal off
            self._off[name] = (off, n)
            off += (n + 3) // 4 * 4  # keep every segment 16-byte aligned

        seg("cu_q", max_seqs + 1)
        seg("seq_slots", max_seqs)
        seg("token_ids", max_tokens)
        seg("positions", max_tokens)
        seg("tok_seq", max_tokens)
        seg("logit_rows", max_tokens)
        for g in range(self.n_groups):
            seg(f"kv_slots{g}", max_tokens)
        for name, planner in self.planners.items():
            seg(f"plan:{name}", planner.words(max_tokens, max_seqs))
        self.front = off  # everything before this goes to the device in one copy per step
        for g in range(self.n_groups):
            seg(f"block_table{g}", max_seqs * self.table_len[g])
        self.total = off
        pin = device.type == "cuda"
        self.host = torch.zeros(self.total, dtype=torch.int32, pin_memory=pin)
        self.host_np = self.host.numpy()
        self.dev = torch.zeros(self.total, dtype=torch.int32, device=device)
        self._copied = torch.cuda.Event() if pin else None
        self._copy_pending = False
        self.copied_words = 0  # int32 words the last build sent to the device
        self.words_sent = 0    # and all builds so far
        # what each block-table row of the host buffer holds: (admission serial, entries written),
        # so that a request that keeps its row from step to step only appends its new pages
        self._row_owner: list[list[tuple[int, int] | None]] = [
            [None] * max_seqs for _ in range(self.n_groups)]
        # views of the two buffers are made once per distinct set of sizes: slicing a torch
        # tensor costs more than filling a decode step's numbers
        self._host_views: dict[str, np.ndarray] = {}
        self._device_views: dict[tuple, dict] = {}
        self._plan_dev = {name: self._d(f"plan:{name}") for name in self.planners}
        self._plan_host = {name: self._h(f"plan:{name}") for name in self.planners}
        self._front_dev, self._front_host = self.dev[:self.front], self.host[:self.front]
        self._group_info = [(g, grp, grp.page_size, grp.window is None)
                            for g, grp in enumerate(cache.groups)]
        self._host_tables = [self.host[self._off[f"block_table{g}"][0]:][:max_seqs * self.table_len[g]]
                             .view(max_seqs, self.table_len[g]) for g in range(self.n_groups)]
        self._dev_tables = [self._d(f"block_table{g}").view(max_seqs, self.table_len[g])
                            for g in range(self.n_groups)]

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
        tables = [self._h(f"block_table{g}").reshape(self.max_seqs, self.table_len[g])
                  for g in range(self.n_groups)]
        kv_slots = [self._h(f"kv_slots{g}") for g in range(self.n_groups)]
        dirty: list[list[tuple[int, int, int]]] = [[] for _ in range(self.n_groups)]  # (row, lo, hi)

        t = 0; r = 0
        q_lens: list[int] = []; kv_lens: list[int] = []; first: list[int] = []
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
            serial = cache.admission(e.request)
            for g, grp, ps, keeps_all in self._group_info:
                table = cache.block_table(e.request, g)
                n_pages = len(table)
                owner = self._row_owner[g][s]
                if keeps_all and owner is not None and owner[0] == serial and owner[1] <= n_pages:
                    if owner[1] < n_pages:
                        tables[g][s, owner[1]:n_pages] = table[owner[1]:]   # only the new pages
                        dirty[g].append((s, owner[1], n_pages))
                        self._row_owner[g][s] = (serial, n_pages)
                else:
                    tables[g][s, :n_pages] = table
                    dirty[g].append((s, 0, n_pages))
                    self._row_owner[g][s] = (serial, n_pages)
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
            q_lens.append(n); kv_lens.append(end); first.append(start)
            t += n
            cu_q[s + 1] = t
        for k in range(pad):  # padding rows: one token at position 0 on the scratch page
            s = S + k
            token_ids[t] = 0; positions[t] = 0; tok_seq[t] = s
            seq_slots[s] = cache.scratch_slot
            for g, grp in enumerate(cache.groups):
                if self._row_owner[g][s] != (-1, 1):
                    tables[g][s, 0] = grp.scratch_page
                    dirty[g].append((s, 0, 1))
                    self._row_owner[g][s] = (-1, 1)   # no admission has serial -1
                kv_slots[g][t] = grp.scratch_page * grp.page_size
            logit_rows[r] = t; r += 1
            q_lens.append(1); kv_lens.append(1); first.append(0)
            t += 1
            cu_q[s + 1] = t
        S += pad; N = t
        plans = {name: planner.plan(self._plan_host[name], self._plan_dev[name], q_lens, first)
                 for name, planner in self.planners.items()}

        self._front_dev.copy_(self._front_host, non_blocking=True)
        self.copied_words = self.front
        for g in range(self.n_groups):
            spans = dirty[g]
            if not spans:
                continue
            lo_row, hi_row = min(x[0] for x in spans), max(x[0] for x in spans) + 1
            if len(spans) > _FEW_ROWS and (hi_row - lo_row) * self.table_len[g] <= _ONE_COPY_WORDS:
                # many rows changed (requests moved): whole rows are contiguous, one copy
                self._dev_tables[g][lo_row:hi_row].copy_(self._host_tables[g][lo_row:hi_row],
                                                         non_blocking=True)
                self.copied_words += (hi_row - lo_row) * self.table_len[g]
            else:
                for s, lo, hi in spans:
                    self._dev_tables[g][s, lo:hi].copy_(self._host_tables[g][s, lo:hi],
                                                        non_blocking=True)
                    self.copied_words += hi - lo
        self.words_sent += self.copied_words
        if self._copied is not None:
            self._copied.record()
            self._copy_pending = True

        sizes = (N, S, r)
        views = self._device_views.get(sizes)
        if views is None:
            if len(self._device_views) >= 512:
                self._device_views.clear()
            views = self._device_views[sizes] = dict(
                token_ids=self._d("token_ids", N), positions=self._d("positions", N),
                tok_seq=self._d("tok_seq", N),
                kv_slots=[self._d(f"kv_slots{g}", N) for g in range(self.n_groups)],
                cu_q=self._d("cu_q", S + 1), seq_slots=self._d("seq_slots", S),
                block_tables=[self._dev_tables[g][:S] for g in range(self.n_groups)],
                logit_rows=self._d("logit_rows", r))
        return StepContext(
            n_tokens=N, n_seqs=S, num_logit_rows=r, max_kv_len=max(kv_lens) if kv_lens else 0,
            max_q_len=max(q_lens) if q_lens else 0, max_seqs=self.max_seqs, ws=ws, q_lens=q_lens,
            kv_lens=kv_lens, plans=plans, **views,
        )
