"""Each CUDA kernel alone against its plain torch twin, at sizes other than the engine's."""

import math
import types

import pytest
import torch

from tests import plain_llama, twin_ops

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from simple_inference_b200 import ops as o
    return o


def dev():
    return torch.device("cuda")


def gen(seed):
    return torch.Generator(device="cuda").manual_seed(seed)


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,h", [(7, 120), (33, 3072), (3, 50), (1, 16400)])
def test_embedding_rmsnorm_swiglu(ops, dt, n, h):
    g = gen(1)
    table = torch.randn(300, h, device=dev(), generator=g).to(dt)
    ids = torch.randint(0, 300, (n,), device=dev(), dtype=torch.int32)
    a, b = torch.empty(n, h, device=dev()), torch.empty(n, h, device=dev())
    ops.embed_gather(table, ids, a)
    twin_ops.embed_gather(table, ids, b)
    assert torch.equal(a, b)

    res = torch.randn(n, h, device=dev(), generator=g)
    delta = torch.randn(n, h, device=dev(), generator=g).to(dt)
    gain = 1 + 0.1 * torch.randn(h, device=dev(), generator=g)
    tol = 2e-6 if dt == torch.float32 else 2e-2      # one bfloat16 ulp at magnitude ~4
    for wdt in (torch.float32, torch.bfloat16):
        o1, o2 = torch.empty(n, h, device=dev(), dtype=dt), torch.empty(n, h, device=dev(), dtype=dt)
        r1, r2 = res.clone(), res.clone()
        ops.rmsnorm(r1, gain.to(wdt), 1e-5, o1, delta=delta)
        twin_ops.rmsnorm(r2, gain.to(wdt), 1e-5, o2, delta=delta)
        assert torch.equal(r1, r2), "the residual add is exact in float32"
        assert (o1.float() - o2.float()).abs().max() < tol
    rows = torch.tensor([n - 1, 0, n // 2], device=dev(), dtype=torch.int32)
    o1, o2 = torch.empty(3, h, device=dev(), dtype=dt), torch.empty(3, h, device=dev(), dtype=dt)
    r1 = res.clone()
    ops.rmsnorm(r1, gain, 3e-6, o1, delta=delta, rows=rows)
    twin_ops.rmsnorm(res.clone(), gain, 3e-6, o2, delta=delta, rows=rows)
    assert torch.equal(r1, res), "with rows given the residual is left alone"
    assert (o1.float() - o2.float()).abs().max() < tol

    gu = torch.randn(n, 2 * h, device=dev(), generator=g).to(dt)
    o1, o2 = torch.empty(n, h, device=dev(), dtype=dt), torch.empty(n, h, device=dev(), dtype=dt)
    ops.swiglu(gu, o1)
    twin_ops.swiglu(gu, o2)
    assert (o1.float() - o2.float()).abs().max() < tol


@pytest.mark.parametrize("m,n,k", [(1, 50, 33), (65, 130, 100), (200, 331, 120), (3, 128256, 64)])
def test_float32_matrix_product_is_true_float32_and_row_invariant(ops, m, n, k):
    g = gen(2)
    a = torch.randn(m, k, device=dev(), generator=g)
    w = torch.randn(n, k, device=dev(), generator=g)
    out = torch.empty(m, n, device=dev())
    ops.linear(a, w, out)
    ref = a.double() @ w.double().T
    # a TF32 product would be off by ~1e-3 * sqrt(k); float32 stays near 1e-6 * sqrt(k)
    assert (out.double() - ref).abs().max() < 4e-6 * math.sqrt(k) * 4
    one = torch.empty(1, n, device=dev())
    ops.linear(a[m // 2:m // 2 + 1].contiguous(), w, one)
    assert torch.equal(one[0], out[m // 2]), "a row's result does not depend on the other rows"


def test_bfloat16_matrix_product_with_float32_output(ops):
    g = gen(3)
    a = torch.randn(5, 96, device=dev(), generator=g).bfloat16()
    w = torch.randn(331, 96, device=dev(), generator=g).bfloat16()
    out = torch.empty(5, 331, device=dev())
    ops.linear(a, w, out)
    assert (out - a.float() @ w.float().T).abs().max() < 1e-3


def paged_case(lens_q, starts, ps, hq, hkv, d, dt, seed=0):
    """A batch of sequences: q_len new tokens after `start` tokens already in the cache."""
    g = gen(seed)
    S, N = len(lens_q), sum(lens_q)
    kv = [s + q for s, q in zip(starts, lens_q)]
    maxp = max((x + ps - 1) // ps for x in kv)
    P = sum((x + ps - 1) // ps for x in kv) + 2
    perm = torch.randperm(P, generator=torch.Generator().manual_seed(seed)).tolist()
    bt = torch.full((S, maxp), -1, dtype=torch.int32)
    tok_seq, pos, slots, cu = [], [], [], [0]
    pi = 0
    for s in range(S):
        for lp in range((kv[s] + ps - 1) // ps):
            bt[s, lp] = perm[pi]
            pi += 1
        for p in range(starts[s], kv[s]):
            tok_seq.append(s)
            pos.append(p)
            slots.append(int(bt[s, p // ps]) * ps + p % ps)
        cu.append(cu[-1] + lens_q[s])
    from simple_inference_b200.engine.batch import Workspace
    from simple_inference_b200.parts.attention_plan import plan_on_device
    I = lambda x: torch.tensor(x, dtype=torch.int32, device=dev())  # noqa: E731
    pool = torch.randn(P + 1, 2, hkv, ps, d, device=dev(), generator=g).to(dt)
    qkv = torch.randn(N, (hq + 2 * hkv) * d, device=dev(), generator=g).to(dt)
    ctx = types.SimpleNamespace(
        block_tables=[bt.to(dev())], tok_seq=I(tok_seq), positions=I(pos), cu_q=I(cu),
        kv_slots=[I(slots)], max_kv_len=max(kv), max_q_len=max(lens_q), max_seqs=S,
        ws=Workspace(dev(), N), plan=plan_on_device(lens_q, starts, dev()))
    return qkv, pool, ctx, N


def assert_attention_close(out, ref, what=""):
    """bfloat16 attention against float32 attention of the same bfloat16 inputs: the kernel
    rounds P to bfloat16 before P V and the result once, so a row may differ by a few 2^-9 of
    its own size.  The bound is relative to each row's RMS, which a wrong or missing key (a
    dropped split, a window one key off) exceeds by far."""
    out, ref = out.float(), ref.float()
    assert bool(torch.isfinite(out).all()), f"{what}: not finite"
    rms = ref.pow(2).mean(dim=-1, keepdim=True).sqrt()
    worst = ((out - ref).abs() / (rms + 1e-6)).max()
    assert worst < ATTENTION_REL_TOL, f"{what}: error {float(worst):.4f} of the row's RMS"


ATTENTION_REL_TOL = 0.04


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hq,hkv,d,ps", [(4, 2, 16, 4), (6, 3, 48, 8), (3, 1, 32, 16),
                                          (24, 8, 128, 16), (2, 2, 256, 2), (5, 5, 80, 3)])
def test_rope_and_page_write(ops, dt, hq, hkv, d, ps):
    qkv, pool, ctx, n = paged_case([37, 1, 300], [0, 90, 11], ps, hq, hkv, d, dt)
    inv = plain_llama.rope_frequencies(d, 10000.0, None).to(dev())
    pool.zero_()
    pool2 = pool.clone()
    q1, q2 = qkv.clone(), qkv.clone()
    ops.rope_kv_store(q1, ctx.positions, inv, ctx.kv_slots[0], pool, hq, hkv, d, ps, True)
    twin_ops.rope_kv_store(q2, ctx.positions, inv, ctx.kv_slots[0], pool2, hq, hkv, d, ps, True)
    tol = 2e-6 if dt == torch.float32 else 4e-2
    assert (q1.float() - q2.float()).abs().max() < tol
    assert (pool.float() - pool2.float()).abs().max() < tol
    assert torch.equal(pool[-1], pool2[-1]) and float(pool[-1].abs().sum()) == 0   # scratch untouched
    q3 = qkv.clone()
    before = pool.clone()
    ops.rope_kv_store(q3, ctx.positions, inv, None, None, hq, hkv, d, ps, False)
    assert torch.equal(q3[:, :hq * d], q1[:, :hq * d]) and torch.equal(pool, before)


@pytest.mark.parametrize("hq,hkv,d,ps,hidden,lens,starts", [
    (4, 2, 16, 4, 64, [1, 1, 1], [0, 90, 11]), (6, 3, 48, 8, 120, [1] * 8, [5, 0, 300, 7, 63, 64, 2, 9]),
    (24, 8, 128, 16, 3072, [1] * 5, [2047, 0, 15, 16, 700]), (5, 5, 80, 3, 200, [7, 2, 1, 3, 3], [0, 40, 3, 8, 100]),
    (2, 2, 256, 2, 72, [1, 2], [100, 3]), (3, 1, 32, 16, 96, [9], [20])])
def test_projection_with_rotation_and_page_write_in_one_kernel(ops, hq, hkv, d, ps, hidden, lens, starts):
    """Up to 16 tokens: the stacked projection, the rotation and the cache write as one kernel
    against the two kernels apart (same arithmetic) and against the float32 twin."""
    dt = torch.bfloat16
    qkv, pool, ctx, n = paged_case(lens, starts, ps, hq, hkv, d, dt)
    assert n <= 16
    g = torch.Generator().manual_seed(n * 31 + d)
    x = torch.randn(n, hidden, generator=g).to(dev(), dt)
    w = (torch.randn((hq + 2 * hkv) * d, hidden, generator=g) / math.sqrt(hidden)).to(dev(), dt)
    inv = plain_llama.rope_frequencies(d, 10000.0, None).to(dev())
    pool.zero_()
    pool_apart, pool_twin = pool.clone(), pool.clone()
    assert ops.can_fuse_projection_rope(x, w, qkv)
    fused = torch.zeros_like(qkv)
    ops.linear_rope_kv_store(x, w, fused, ctx.positions, inv, ctx.kv_slots[0], pool, hq, hkv, d, ps, True)
    apart = torch.empty_like(qkv)
    ops.linear(x, w, apart)
    projected = apart.clone()
    ops.rope_kv_store(apart, ctx.positions, inv, ctx.kv_slots[0], pool_apart, hq, hkv, d, ps, True)
    q = slice(0, hq * d)
    assert (fused[:, q].float() - apart[:, q].float()).abs().max() <= 2 ** -7 * apart[:, q].float().abs().max()
    assert (fused[:, q] != apart[:, q]).float().mean() < 0.01      # one rounding of a sum apart at most
    assert (pool.float() - pool_apart.float()).abs().max() <= 2 ** -7 * pool_apart.float().abs().max()
    assert (pool != pool_apart).float().mean() < 0.01
    assert float(fused[:, hq * d:].abs().sum()) == 0                # keys and values go to the pages only
    assert float(pool[-1].abs().sum()) == 0                          # scratch untouched
    twin = projected.clone()
    twin_ops.rope_kv_store(twin, ctx.positions, inv, ctx.kv_slots[0], pool_twin, hq, hkv, d, ps, True)
    assert (fused[:, q].float() - twin[:, q].float()).abs().max() < 4e-2
    assert (pool.float() - pool_twin.float()).abs().max() < 4e-2
    # without the write only the queries come out
    before = pool.clone()
    again = torch.zeros_like(qkv)
    ops.linear_rope_kv_store(x, w, again, ctx.positions, inv, None, None, hq, hkv, d, ps, False)
    assert torch.equal(again, fused) and torch.equal(pool, before)


@pytest.mark.parametrize("hq,hkv,d,ps,window", [(4, 2, 16, 4, None), (6, 3, 48, 8, None),
                                                 (3, 1, 32, 16, 7), (24, 8, 128, 16, None),
                                                 (2, 2, 256, 2, None), (5, 5, 80, 3, 33)])
def test_generic_attention_float32(ops, hq, hkv, d, ps, window):
    qkv, pool, ctx, n = paged_case([37, 1, 300, 2], [0, 90, 11, 513], ps, hq, hkv, d, torch.float32)
    o1, o2 = torch.empty(n, hq * d, device=dev()), torch.empty(n, hq * d, device=dev())
    ops.attention_generic(qkv, pool, ctx.block_tables[0], ctx.tok_seq, ctx.positions, o1, hq, hkv,
                          d, 1 / math.sqrt(d), window)
    twin_ops.attention_generic(qkv, pool, ctx.block_tables[0], ctx.tok_seq, ctx.positions, o2, hq,
                               hkv, d, 1 / math.sqrt(d), window)
    assert (o1 - o2).abs().max() < 5e-6


CASES = [
    ("tile of 64", [64], [0], 16, 4, 2, 128, None, None),
    ("ragged portions", [37, 200, 2], [0, 0, 5], 4, 4, 2, 16, None, None),
    ("portions deep in a context", [130, 70], [33, 500], 16, 24, 8, 128, None, None),
    ("head size 48, three groups", [100, 3], [0, 77], 8, 6, 3, 48, None, None),
    ("window over a tile edge", [65], [100], 16, 3, 1, 32, 40, None),
    ("head size 256, page of 2", [300], [0], 2, 2, 2, 256, None, None),
    ("first token", [1], [0], 16, 4, 2, 128, None, None),
    ("decode at three depths", [1, 1, 1], [5, 300, 63], 16, 24, 8, 128, None, None),
    ("decode, one split", [1, 1], [2047, 64], 16, 24, 8, 128, None, 1),
    ("decode, seven splits", [1, 1], [2047, 64], 16, 24, 8, 128, None, 7),
    ("decode, more splits than tiles", [1, 1], [100, 3], 16, 24, 8, 128, None, 32),
    ("decode, tiny heads", [1, 1, 1, 1], [0, 1, 100, 17], 4, 4, 2, 16, None, None),
    ("decode with a window", [1, 1], [200, 30], 8, 6, 3, 48, 50, None),
    ("twenty heads per group", [1], [500], 16, 40, 2, 64, None, None),
    ("decode, head size 256", [1], [1000], 2, 2, 2, 256, None, None),
    ("portions beside decode tokens", [1, 50, 1, 2, 129], [100, 10, 0, 40, 0], 16, 24, 8, 128, None, None),
]


@pytest.mark.parametrize("what,lens,starts,ps,hq,hkv,d,window,splits", CASES,
                         ids=[c[0] for c in CASES])
def test_tensor_core_attention_bfloat16(ops, monkeypatch, what, lens, starts, ps, hq, hkv, d,
                                        window, splits):
    qkv, pool, ctx, n = paged_case(lens, starts, ps, hq, hkv, d, torch.bfloat16)
    if splits:
        monkeypatch.setattr(ops, "plan_kv_splits", lambda *a: splits)
    out = torch.zeros(n, hq * d, device=dev(), dtype=torch.bfloat16)
    ops.paged_attention(qkv, pool, ctx, ctx.plan, 0, out, hq, hkv, d, 1 / math.sqrt(d), window)
    ref = torch.zeros(n, hq * d, device=dev())
    twin_ops.attention_generic(qkv.float(), pool.float(), ctx.block_tables[0], ctx.tok_seq,
                               ctx.positions, ref, hq, hkv, d, 1 / math.sqrt(d), window)
    assert_attention_close(out, ref, what)


WIDE_CASES = [
    ("one full tile", [128], [0], 16, 4, 2, None),
    ("short tile", [70], [0], 16, 4, 2, None),
    ("six key tiles, ragged end", [700], [0], 16, 6, 3, None),
    ("deep in a context, page of 8", [130, 66], [333, 1500], 8, 4, 1, None),
    ("page of 64", [200], [77], 64, 2, 2, None),
    ("page of 32, three portions", [64, 300, 2], [0, 31, 900], 32, 3, 3, None),
    ("window inside one tile", [300], [100], 16, 4, 2, 40),
    ("window over several tiles", [260], [1000], 16, 2, 1, 300),
    ("twenty-four heads", [256], [0], 16, 24, 8, None),
]


@pytest.mark.parametrize("d", [128, 64])
@pytest.mark.parametrize("what,lens,starts,ps,hq,hkv,window", WIDE_CASES,
                         ids=[c[0] for c in WIDE_CASES])
def test_tcgen05_prefill_attention(ops, what, lens, starts, ps, hq, hkv, window, d):
    qkv, pool, ctx, n = paged_case(lens, starts, ps, hq, hkv, d, torch.bfloat16, seed=3)
    assert ops.wide_prefill_fits(ctx.plan, d, ps)
    out = torch.zeros(n, hq * d, device=dev(), dtype=torch.bfloat16)
    ops.attention_prefill_wide(qkv[:, :hq * d], pool, ctx, ctx.plan, 0, out, hq, hkv, d,
                               1 / math.sqrt(d), window)
    ref = torch.zeros(n, hq * d, device=dev())
    twin_ops.attention_generic(qkv.float(), pool.float(), ctx.block_tables[0], ctx.tok_seq,
                               ctx.positions, ref, hq, hkv, d, 1 / math.sqrt(d), window)
    assert bool(torch.isfinite(out.float()).all()), "a bounded wait ran out (NaN marks it)"
    assert_attention_close(out, ref, what)


@pytest.mark.parametrize("d", [128, 64])
def test_tcgen05_prefill_finds_one_far_key(ops, d):
    """One key per query head, far back and on a page of its own, matches 30 times better
    than the rest: every row's output must be that key's value (7)."""
    hq, hkv, ps = 4, 2, 16
    qkv, pool, ctx, n = paged_case([200, 129], [900, 300], ps, hq, hkv, d, torch.bfloat16, seed=5)
    pool.mul_(0.05)
    table = ctx.block_tables[0]
    for seq, far in ((0, 437), (1, 23)):
        page, off = int(table[seq, far // ps]), far % ps
        toks = (ctx.tok_seq == seq).nonzero().flatten()
        for h in range(hq):
            kvh = h // (hq // hkv)
            pool[page, 0, kvh, off, h * 3] = 30.0
            key = torch.zeros(d, device=dev())
            key[h * 3] = 30.0
            qkv[toks, h * d:(h + 1) * d] = key.bfloat16()
        pool[page, 1, :, off, :] = 7.0
    out = torch.zeros(n, hq * d, device=dev(), dtype=torch.bfloat16)
    ops.attention_prefill_wide(qkv[:, :hq * d], pool, ctx, ctx.plan, 0, out, hq, hkv, d,
                               1 / math.sqrt(d), None)
    assert (out.float() - 7.0).abs().max() < 0.1


def test_attention_finds_one_far_key_among_hundreds(ops):
    """Random keys give flat softmax rows that hide a wrong page.  Here one far key (on a
    page of its own, in the middle of the table) matches the query 30 times better than the
    rest, so the output must be that key's value."""
    hq, hkv, d, ps = 4, 2, 64, 16
    for dt in (torch.float32, torch.bfloat16):
        qkv, pool, ctx, n = paged_case([1, 70], [900, 700], ps, hq, hkv, d, dt, seed=5)
        pool.mul_(0.05)
        table = ctx.block_tables[0]
        for seq, far in ((0, 437), (1, 23)):
            page, off = int(table[seq, far // ps]), far % ps
            toks = (ctx.tok_seq == seq).nonzero().flatten()
            for h in range(hq):
                kvh = h // (hq // hkv)
                key = torch.zeros(d, device=dev())
                key[h * 3] = 30.0
                pool[page, 0, kvh, off, h * 3] = 30.0
                qkv[toks, h * d:(h + 1) * d] = key.to(dt) * 1.0
            pool[page, 1, :, off, :] = 7.0
        out = torch.zeros(n, hq * d, device=dev(), dtype=dt)
        ops.paged_attention(qkv, pool, ctx, ctx.plan, 0, out, hq, hkv, d, 1 / math.sqrt(d), None)
        assert (out.float() - 7.0).abs().max() < 0.1, f"{dt}: the far key was not found"


def _plant_key(qkv, pool, ctx, seq, far, hq, hkv, d, ps, dt):
    """Make key `far` of sequence `seq` match every query of that sequence 30 times better than
    any other key, and give it the value 7."""
    table = ctx.block_tables[0]
    page, off = int(table[seq, far // ps]), far % ps
    toks = (ctx.tok_seq == seq).nonzero().flatten()
    for h in range(hq):
        kvh = h // (hq // hkv)
        key = torch.zeros(d, device=dev())
        key[h * 3] = 30.0
        pool[page, 0, kvh, off, h * 3] = 30.0
        qkv[toks, h * d:(h + 1) * d] = key.to(dt)
    pool[page, 1, :, off, :] = 7.0


@pytest.mark.parametrize("splits", [7, 32])
def test_split_decode_attention_finds_one_far_key(ops, monkeypatch, splits):
    """The TMA-fed decode kernel at head size 128 with its keys cut into 7 and 32 splits: the
    one key that matters lies in one split, and the join must weigh that split's part."""
    hq, hkv, d, ps = 24, 8, 128, 16
    monkeypatch.setattr(ops, "plan_kv_splits", lambda *a: splits)
    for fars in ((437, 23), (2040, 1000), (0, 1999)):
        qkv, pool, ctx, n = paged_case([1, 1], [2047, 2000], ps, hq, hkv, d, torch.bfloat16, seed=7)
        pool.mul_(0.05)
        for seq, far in enumerate(fars):
            _plant_key(qkv, pool, ctx, seq, far, hq, hkv, d, ps, torch.bfloat16)
        out = torch.zeros(n, hq * d, device=dev(), dtype=torch.bfloat16)
        ops.paged_attention(qkv, pool, ctx, ctx.plan, 0, out, hq, hkv, d, 1 / math.sqrt(d), None)
        assert (out.float() - 7.0).abs().max() < 0.1, f"keys {fars} with {splits} splits"


WINDOW_EDGE_CASES = [
    # what, head size, page, window, (start, tokens) of the sequences, position of the planted key
    ("decode by TMA, head 128", 128, 16, 40, [(139, 1), (140, 1)], 100),
    ("decode by TMA, window over many tiles", 128, 16, 300, [(1299, 1), (1300, 1)], 1000),
    ("decode, head 48", 48, 8, 50, [(249, 1), (250, 1)], 200),
    ("mma.sync portions, head 64", 64, 16, 40, [(120, 70)], 100),
    ("mma.sync portions, window over a tile edge", 32, 16, 70, [(130, 100)], 100),
    ("tcgen05 portions, head 128", 128, 16, 40, [(100, 200)], 130),
    ("tcgen05 portions, window over several tiles", 128, 16, 300, [(900, 260)], 700),
]


@pytest.mark.parametrize("what,d,ps,window,seqs,far", WINDOW_EDGE_CASES,
                         ids=[c[0] for c in WINDOW_EDGE_CASES])
def test_the_window_ends_exactly_where_it_should(ops, what, d, ps, window, seqs, far):
    """A query at position p sees the keys at p-window+1 .. p.  One key matches every query
    30 times better than the rest and carries the value 7: rows whose window still holds it
    must return 7, rows whose window has just passed it must not see it at all.  Random keys
    would hide an edge that is off by one (one key among `window` moves a row by 1/window)."""
    hq, hkv = 4, 2
    lens, starts = [n for _, n in seqs], [s for s, _ in seqs]
    qkv, pool, ctx, n = paged_case(lens, starts, ps, hq, hkv, d, torch.bfloat16, seed=9)
    pool.mul_(0.05)
    for seq in range(len(seqs)):
        _plant_key(qkv, pool, ctx, seq, far, hq, hkv, d, ps, torch.bfloat16)
    out = torch.zeros(n, hq * d, device=dev(), dtype=torch.bfloat16)
    ops.paged_attention(qkv, pool, ctx, ctx.plan, 0, out, hq, hkv, d, 1 / math.sqrt(d), window)
    pos = ctx.positions.tolist()
    sees = torch.tensor([far <= p <= far + window - 1 for p in pos], device=dev())
    assert bool(sees.any()) and bool((~sees).any()), "the case must have rows on both sides"
    err = (out.float() - 7.0).abs().amax(dim=-1)
    assert float(err[sees].max()) < 0.1, "a row whose window holds the key did not find it"
    assert float(out.float().abs().amax(dim=-1)[~sees].max()) < 1.0, \
        "a row whose window has passed the key still saw it"
    ref = torch.zeros(n, hq * d, device=dev())
    twin_ops.attention_generic(qkv.float(), pool.float(), ctx.block_tables[0], ctx.tok_seq,
                               ctx.positions, ref, hq, hkv, d, 1 / math.sqrt(d), window)
    assert (out.float() - ref).abs().max() < 2e-2


def test_sampling_kernel_against_plain_sampler(ops):
    V = 1000
    logits = torch.randn(8, V, device=dev(), generator=gen(5)) * 3
    logits[7, 10] = logits[7, 20] = logits[7].max() + 1            # a tie: lower index wins
    temp = torch.tensor([0, 1.0, 0.8, 0.8, 0.8, 1.3, 2.0, 0], device=dev())
    top_k = torch.tensor([0, 0, 50, 0, 20, 5, 1, 0], device=dev(), dtype=torch.int32)
    top_p = torch.tensor([1.0, 1.0, 1.0, 0.9, 0.5, 0.0, 1.0, 1.0], device=dev())
    seed = torch.arange(1, 9, device=dev(), dtype=torch.int32)
    sid = torch.arange(9, 1, -1, device=dev(), dtype=torch.int32)
    ctr = torch.arange(0, 8, device=dev(), dtype=torch.int32)
    got = torch.empty(8, device=dev(), dtype=torch.int32)
    ops.sample(logits, temp, top_k, top_p, seed, sid, ctr, got)
    want = torch.empty(8, dtype=torch.int32)
    twin_ops.sample(logits.cpu(), temp.cpu(), top_k.cpu(), top_p.cpu(), seed.cpu(), sid.cpu(),
                    ctr.cpu(), want)
    assert got.cpu().tolist() == want.tolist()
    assert int(got[7]) == 10 and int(got[0]) == int(logits[0].argmax())
    # a vocabulary that is no power of two and far larger than the block
    big = torch.randn(2, 128256, device=dev(), generator=gen(6))
    t2 = torch.tensor([0.0, 0.7], device=dev())
    k2 = torch.tensor([0, 40], device=dev(), dtype=torch.int32)
    p2 = torch.tensor([1.0, 0.95], device=dev())
    z = torch.zeros(2, device=dev(), dtype=torch.int32)
    got = torch.empty(2, device=dev(), dtype=torch.int32)
    ops.sample(big, t2, k2, p2, z, z, z, got)
    assert int(got[0]) == int(big[0].argmax())
    kept = torch.isfinite(plain_llama.filter_logits(big[1].cpu(), 0.7, 40, 0.95))
    assert bool(kept[int(got[1])])
    # greedy rows read 16 bytes at a time where they can: ties go to the lowest index, a row of
    # NaN gives -1, rows that start off a 16-byte boundary and widths that are no multiple of 4
    for vocab, ld in ((128256, 128256), (5003, 5003), (5003, 5004), (7, 7), (4099, 4100)):
        rows = torch.randn(5, ld, device=dev(), generator=gen(vocab))
        rows[1, :vocab] = float("nan")
        rows[2, :vocab] = 0.25                      # all equal: index 0
        rows[3, vocab - 1] = 50.0                   # the last one, in the scalar tail
        rows[4, [3, vocab // 2, vocab - 2]] = 60.0  # a tie: the first of them
        if ld > vocab:
            rows[:, vocab:] = 1000.0                # beyond the vocabulary: never read
        zero = torch.zeros(5, device=dev())
        zi = torch.zeros(5, device=dev(), dtype=torch.int32)
        got = torch.empty(5, device=dev(), dtype=torch.int32)
        ops.sample(rows[:, :vocab], zero, zi, torch.ones(5, device=dev()), zi, zi, zi, got)
        assert got.tolist() == [int(rows[0, :vocab].argmax()), -1, 0, vocab - 1, 3], (vocab, ld)


def test_kernels_refuse_what_they_cannot_take(ops):
    x = torch.zeros(4, 40, device=dev())
    with pytest.raises(ops.KernelError):
        ops.embed_gather(torch.zeros(10, 40), torch.zeros(4, dtype=torch.int32), torch.zeros(4, 40))
    with pytest.raises(ops.KernelError):
        ops.linear(x, torch.zeros(8, 41, device=dev()), torch.zeros(4, 8, device=dev()))
    with pytest.raises(ops.KernelError):
        ops.attention_library(40)            # head sizes come in steps of 16
    with pytest.raises(ops.KernelError):
        ops.rmsnorm(x, torch.ones(40, device=dev()), 1e-5, torch.zeros(4, 40, device=dev()),
                    rows=torch.zeros(4, device=dev(), dtype=torch.int64))


@pytest.mark.parametrize("m", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("n,k", [(50, 64), (331, 120), (5120, 3072), (16, 8), (3072, 8192)])
def test_weight_streaming_product_for_few_rows(ops, m, n, k):
    """The hand-written product that decode steps use (M <= 16), all three epilogues."""
    g = gen(7)
    x = (torch.randn(m, k, device=dev(), generator=g) * 0.5).bfloat16()
    w = (torch.randn(2 * n, k, device=dev(), generator=g) * 0.1).bfloat16()
    ref = x.float() @ w.float().T                       # [m, 2n]
    scale = max(1.0, float(ref.abs().max()))
    assert ops.can_fuse_swiglu(x, w)
    out = torch.empty(m, 2 * n, device=dev(), dtype=torch.bfloat16)
    ops.linear(x, w, out)
    assert (out.float() - ref).abs().max() < 8e-3 * scale      # one bfloat16 rounding of the result
    out32 = torch.empty(m, 2 * n, device=dev())
    ops.linear(x, w, out32)
    assert (out32 - ref).abs().max() < 1e-4 * scale            # float32 accumulation, no rounding
    fused = torch.empty(m, n, device=dev(), dtype=torch.bfloat16)
    ops.linear_swiglu(x, w, fused)
    gate, up = ref[:, :n], ref[:, n:]
    want = gate * torch.sigmoid(gate) * up
    assert (fused.float() - want).abs().max() < 8e-3 * max(1.0, float(want.abs().max()))
    # a row's result does not depend on how many rows ride along
    one = torch.empty(1, 2 * n, device=dev())
    ops.linear(x[m - 1:m], w, one)
    assert torch.equal(one[0], out32[m - 1])


@pytest.mark.parametrize("m,n,k", [(8, 3072, 3072), (3, 400, 2048), (16, 3072, 8192), (5, 50, 64),
                                   (1, 1000, 1024), (9, 200, 5000)])
def test_product_cut_along_k_and_the_norm_that_adds_its_slices(ops, m, n, k):
    """Products that feed the residual stream may leave their sum to the RMSNorm that follows:
    float32 slices, one per k-range, added in a fixed order.  The norm given the slices must do
    exactly what it does given the rounded sum."""
    from simple_inference_b200.engine.batch import Workspace
    g = gen(11)
    x = (torch.randn(m, k, device=dev(), generator=g) * 0.5).bfloat16()
    w = (torch.randn(n, k, device=dev(), generator=g) * 0.1).bfloat16()
    ref = x.float() @ w.float().T
    ws = Workspace(dev(), 64)
    parts = ops.linear_for_residual(x, w, ws, "t", True)
    splits = ops.core().si_gemm_skinny_splits(n, k)
    assert splits == (1 if k < 1024 else splits) and 1 <= splits <= ops.SKINNY_MAX_SPLITS
    assert splits > 1 or (n, k) == (50, 64), "the larger cases here are all cut"
    if splits == 1:
        assert isinstance(parts, torch.Tensor) and parts.dtype == torch.bfloat16
        assert (parts.float() - ref).abs().max() < 8e-3 * max(1.0, float(ref.abs().max()))
        return
    assert isinstance(parts, ops.PartialSums) and parts.slices.shape == (splits, m, n)
    assert (parts.slices.sum(0) - ref).abs().max() < 1e-4 * max(1.0, float(ref.abs().max()))
    whole = parts.tensor()
    assert whole.dtype == torch.bfloat16
    plain = ops.linear_for_residual(x, w, ws, "u", False)          # the same product, not cut
    assert isinstance(plain, torch.Tensor)
    assert (whole.float() - plain.float()).abs().max() <= 2 ** -7 * float(plain.float().abs().max())
    gain = 1 + 0.1 * torch.randn(n, device=dev(), generator=g)
    res = torch.randn(m, n, device=dev(), generator=g)
    r1, r2 = res.clone(), res.clone()
    o1 = torch.empty(m, n, device=dev(), dtype=torch.bfloat16)
    o2 = torch.empty_like(o1)
    ops.rmsnorm(r1, gain, 1e-5, o1, delta=parts)
    ops.rmsnorm(r2, gain, 1e-5, o2, delta=whole)
    assert torch.equal(r1, r2) and torch.equal(o1, o2)
    rows = torch.tensor([m - 1, 0], device=dev(), dtype=torch.int32)
    o3 = torch.empty(2, n, device=dev(), dtype=torch.bfloat16)
    o4 = torch.empty_like(o3)
    r3 = res.clone()
    ops.rmsnorm(r3, gain, 1e-5, o3, delta=parts, rows=rows)
    ops.rmsnorm(res.clone(), gain, 1e-5, o4, delta=whole, rows=rows)
    assert torch.equal(o3, o4) and torch.equal(r3, res)


@pytest.mark.parametrize("m,n,k", [(256, 512, 64), (300, 264, 72), (257, 40, 8), (2048, 3072, 3072),
                                   (700, 5120, 200)])
def test_tensor_memory_product_on_sm_pairs(ops, m, n, k):
    """The same product with 256-row tiles on clusters of two blocks (tcgen05 cta_group::2),
    against float32 and against the one-block kernel; plain and SwiGLU; ragged edges."""
    g = gen(9)
    x = (torch.randn(m, k, device=dev(), generator=g) * 0.5).bfloat16()
    w = (torch.randn(2 * n, k, device=dev(), generator=g) * 0.1).bfloat16()
    ref = x.float() @ w.float().T
    pair = torch.zeros(m, 2 * n, device=dev(), dtype=torch.bfloat16)
    ops.linear_tc(x, w, pair, paired=True)
    ops.check_status()
    assert (pair.float() - ref).abs().max() < 8e-3 * max(1.0, float(ref.abs().max()))
    single = torch.zeros(m, 2 * n, device=dev(), dtype=torch.bfloat16)
    ops.linear_tc(x, w, single, paired=False)
    ops.check_status()
    assert torch.equal(pair, single), "both kernels add the k-steps in the same order"
    fused = torch.zeros(m, n, device=dev(), dtype=torch.bfloat16)
    ops.linear_tc(x, w, fused, swiglu=True, paired=True)
    ops.check_status()
    gate, up = ref[:, :n], ref[:, n:]
    want = gate * torch.sigmoid(gate) * up
    assert (fused.float() - want).abs().max() < 8e-3 * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("m,n,k,splits", [(256, 512, 512, 2), (300, 264, 1000, 3), (512, 3072, 3072, 3),
                                          (700, 2048, 8192, 8), (257, 40, 2048, 5)])
def test_tensor_memory_product_cut_along_k(ops, m, n, k, splits):
    """The product on pairs of SMs with its k-range cut into float32 slices (for the few-hundred-row
    portions whose tiles do not fill the pairs): the slices add up to the product, and the norm
    given the slices does what it does given their rounded sum."""
    g = gen(12)
    x = (torch.randn(m, k, device=dev(), generator=g) * 0.5).bfloat16()
    w = (torch.randn(n, k, device=dev(), generator=g) * 0.1).bfloat16()
    ref = x.float() @ w.float().T
    slices = torch.full((splits, m, n), float("nan"), device=dev())
    code = ops.core().si_gemm_tc2_partial(
        ops._p(x), x.stride(0), ops._p(w), ops._p(slices), n, m, n, k, splits,
        ops._p(ops.status_tensor(dev())), ops._stream())
    assert code == 0
    ops.check_status()
    assert torch.isfinite(slices).all(), "every element of every slice is written"
    assert (slices.sum(0) - ref).abs().max() < 1e-4 * max(1.0, float(ref.abs().max()))
    parts = ops.PartialSums(slices, torch.bfloat16)
    whole = parts.tensor()
    gain = 1 + 0.1 * torch.randn(n, device=dev(), generator=g)
    res = torch.randn(m, n, device=dev(), generator=g)
    r1, r2 = res.clone(), res.clone()
    o1 = torch.empty(m, n, device=dev(), dtype=torch.bfloat16)
    o2 = torch.empty_like(o1)
    ops.rmsnorm(r1, gain, 1e-5, o1, delta=parts)
    ops.rmsnorm(r2, gain, 1e-5, o2, delta=whole)
    assert torch.equal(r1, r2) and torch.equal(o1, o2)


def test_residual_product_of_a_few_hundred_rows_is_cut_where_it_pays(ops):
    from simple_inference_b200.engine.batch import Workspace
    g = gen(13)
    m, n, k = 512, 3072, 8192
    x = (torch.randn(m, k, device=dev(), generator=g) * 0.5).bfloat16()
    w = (torch.randn(n, k, device=dev(), generator=g) * 0.1).bfloat16()
    ws = Workspace(dev(), 2048)
    got = ops.linear_for_residual(x, w, ws, "t", True)
    ops.check_status()
    splits = ops.core().si_gemm_tc2_splits(m, n, k)
    assert 1 < splits <= 8, "24 tiles for 74 pairs of SMs and 64 stages each: cutting pays"
    assert isinstance(got, ops.PartialSums) and got.slices.shape == (splits, m, n)
    plain = ops.linear_for_residual(x, w, ws, "u", False)
    assert (got.tensor().float() - plain.float()).abs().max() <= 2 ** -6 * float(plain.float().abs().max())
    # a product with tiles enough for every pair is left whole
    assert ops.core().si_gemm_tc2_splits(2048, 16384, 3072) == 1


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (130, 264, 72), (96, 40, 8), (300, 5120, 3072),
                                   (2048, 3072, 8192), (1000, 331 * 8, 120)])
def test_tensor_memory_product_for_many_rows(ops, m, n, k):
    """The tcgen05 product that prompt portions use (M >= 96): TMA loads, accumulators in
    tensor memory; plain and SwiGLU epilogues; ragged edges in every dimension."""
    g = gen(8)
    x = (torch.randn(m, k, device=dev(), generator=g) * 0.5).bfloat16()
    w = (torch.randn(2 * n, k, device=dev(), generator=g) * 0.1).bfloat16()
    ref = x.float() @ w.float().T
    out = torch.zeros(m, 2 * n, device=dev(), dtype=torch.bfloat16)
    ops.linear(x, w, out)                                   # routed to the tcgen05 kernel
    ops.check_status()
    assert (out.float() - ref).abs().max() < 8e-3 * max(1.0, float(ref.abs().max()))
    fused = torch.zeros(m, n, device=dev(), dtype=torch.bfloat16)
    assert ops.can_fuse_swiglu(x, w)
    ops.linear_swiglu(x, w, fused)
    ops.check_status()
    gate, up = ref[:, :n], ref[:, n:]
    want = gate * torch.sigmoid(gate) * up
    assert (fused.float() - want).abs().max() < 8e-3 * max(1.0, float(want.abs().max()))
    # a row's result does not depend on how many rows ride along (same k order for every tile)
    half = torch.zeros(m - 32, 2 * n, device=dev(), dtype=torch.bfloat16)
    ops.linear(x[32:].contiguous(), w, half) if m - 32 >= 96 else None
    if m - 32 >= 96:
        assert torch.equal(half, out[32:])
