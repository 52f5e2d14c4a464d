"""The batch builder on the CPU: the device copy of the step's description is what the host
holds, although block tables travel only by the spans that changed."""

import random

import pytest
import torch

from simple_inference_b200.cache import CacheManager
from simple_inference_b200.engine.batch import BatchBuilder, StepEntry, Workspace
from simple_inference_b200.parts.attention_plan import PagedAttentionPlanner, QUERY_TILE, WIDE_TILE
from simple_inference_b200.parts.base import PagedKVSpec


def _builder(window=None, max_seqs=6, max_tokens=96, max_seq_len=200, page=4, pages=400):
    specs = [PagedKVSpec(2, 16, None), PagedKVSpec(2, 16, window)] if window else [PagedKVSpec(2, 16)]
    cache = CacheManager(specs, page, pages, max_seqs, max_tokens, torch.float32, "cpu")
    builder = BatchBuilder(cache, max_tokens, max_seqs, max_seq_len, torch.device("cpu"),
                           planners={PagedAttentionPlanner.name: PagedAttentionPlanner})
    return cache, builder, Workspace(torch.device("cpu"), max_tokens)


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("window", [None, 9])
def test_device_tables_follow_the_host_through_random_steps(seed, window):
    rng = random.Random(seed)
    cache, builder, ws = _builder(window)
    live: dict[int, int] = {}
    next_id = 0
    sent_tables = 0
    for step in range(120):
        while len(live) < 6 and rng.random() < 0.5:
            total = rng.randint(2, 150)
            cache.admit(next_id, total)
            live[next_id] = total
            next_id += 1
        if not live:
            continue
        chosen = rng.sample(sorted(live), rng.randint(1, len(live)))   # rows move between steps
        rng.shuffle(chosen)
        entries, room = [], builder.max_tokens
        for r in chosen:
            n = min(live[r], rng.choice([1, 1, 1, 2, 7, 33]), room)
            if n <= 0:
                continue
            entries.append(StepEntry(r, [1] * n, [n - 1]))
            live[r] -= n
            room -= n
        if not entries:
            continue
        starts = [cache.extend(e.request, len(e.tokens)) for e in entries]
        decode_only = all(len(e.tokens) == 1 for e in entries)
        pad_to = 6 if decode_only and rng.random() < 0.5 else None
        ctx = builder.build(entries, starts, ws, pad_to=pad_to)
        sent_tables += builder.copied_words - builder.front
        # what the kernels will read: every live entry of every table, the write slots, positions
        for g, grp in enumerate(cache.groups):
            for s, (e, start) in enumerate(zip(entries, starts)):
                table = cache.block_table(e.request, g)
                got = ctx.block_tables[g][s, :len(table)].tolist()
                first_needed = 0 if grp.window is None else max(0, start - grp.window + 1) // grp.page_size
                assert got[first_needed:] == table[first_needed:]
                assert all(p >= 0 for p in table[first_needed:])
                t0 = int(ctx.cu_q[s])
                for i in range(len(e.tokens)):
                    assert int(ctx.kv_slots[g][t0 + i]) == cache.write_slot(e.request, g, start + i)
                    assert int(ctx.positions[t0 + i]) == start + i
            for s in range(len(entries), ctx.n_seqs):    # padding rows sit on the scratch page
                assert int(ctx.block_tables[g][s, 0]) == grp.scratch_page
        assert ctx.q_lens[:len(entries)] == [len(e.tokens) for e in entries]
        plan = ctx.plans[PagedAttentionPlanner.name]
        singles = [s for s, n in enumerate(ctx.q_lens) if n == 1]
        assert plan.single_seqs.tolist() == singles and plan.n_single == len(singles)
        assert plan.n_tiles == sum(-(-n // QUERY_TILE) for n in ctx.q_lens if n > 1)
        assert plan.n_wide == sum(-(-n // WIDE_TILE) for n in ctx.q_lens if n > 1)
        paired = [i for i in plan.tile_pairs.tolist() if i >= 0]
        assert sorted(paired) == list(range(plan.n_tiles))
        for r in [r for r in live if live[r] == 0]:
            cache.release(r)
            del live[r]
        cache.check()
    # far fewer table words travelled than whole tables every step would have cost
    assert sent_tables < 120 * builder.max_seqs * builder.table_len[0] // 2


def test_a_decode_step_sends_only_the_pages_it_gained():
    cache, builder, ws = _builder(max_seq_len=4000, pages=2200)
    for r in range(2):
        cache.admit(r, 4000)
    starts = [cache.extend(r, 45) for r in range(2)]
    builder.build([StepEntry(r, [1] * 45, []) for r in range(2)], starts, ws)
    assert builder.copied_words - builder.front == 2 * 12      # both tables, 12 pages each
    words = []
    for _ in range(8):
        starts = [cache.extend(r, 1) for r in range(2)]
        builder.build([StepEntry(r, [1], [0]) for r in range(2)], starts, ws)
        words.append(builder.copied_words - builder.front)
    assert sum(words) == 2 * 2 and max(words) == 2             # 45 -> 53 tokens: pages 13 and 14 of each
    assert builder.table_len[0] == 1000                        # whole tables would be 2,000 words a step
