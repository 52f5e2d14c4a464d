"""The decode-attention entry point that allocates nothing (csrc/no_alloc.h).

Some users of the library cannot allocate device memory while they run: the GPU's
memory may already belong to one big pool, the allocator's lock and synchronisation
may be off limits in a latency-critical loop, or the caller may sit in another language
behind the C symbols with no torch allocator at hand.  For them the library keeps a
4 MiB scratch array inside its own image.  This test reaches `si_attn_decode_static`
through its exported C symbol, as such a caller would, and checks it against the
ordinary entry point (which takes the caller's scratch) on two calls in a row, the
second with different sizes so that what the first left in the array is still there;
and that a call whose splits need more than the array holds is refused.

The file sorts last on purpose: a run that stops at the first failure has then already
run every other test.
"""

import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

SCRATCH_FLOATS = 1 << 20


def _case(n_seqs, ctx_lens, hq, hkv, d, ps, seed):
    """Sequences with one new token each over `ctx_lens` cached keys: device tensors."""
    dev = torch.device("cuda")
    g = torch.Generator(device="cuda").manual_seed(seed)
    kv = [c + 1 for c in ctx_lens]
    maxp = max((x + ps - 1) // ps for x in kv)
    pages = sum((x + ps - 1) // ps for x in kv)
    perm = torch.randperm(pages, generator=torch.Generator().manual_seed(seed)).tolist()
    table = torch.zeros(n_seqs, maxp, dtype=torch.int32)
    k = 0
    for s in range(n_seqs):
        for lp in range((kv[s] + ps - 1) // ps):
            table[s, lp] = perm[k]
            k += 1
    I = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)  # noqa: E731
    return dict(
        q=torch.randn(n_seqs, (hq + 2 * hkv) * d, device=dev, generator=g).bfloat16(),
        pool=torch.randn(pages + 1, 2, hkv, ps, d, device=dev, generator=g).bfloat16(),
        table=table.to(dev), cu_q=I(list(range(n_seqs + 1))), positions=I(ctx_lens),
        single=I(list(range(n_seqs))), n=n_seqs, hq=hq, hkv=hkv, d=d, ps=ps)


def _call(lib, fn_name, c, out, n_splits, scratch=None):
    P = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    head = [P(c["q"]), c["q"].stride(0), P(c["pool"]), c["pool"].shape[0], P(c["table"]),
            c["table"].stride(0),
            P(c["cu_q"]), P(c["positions"]), P(c["single"]), c["n"], P(out), out.stride(0)]
    tail = [c["hq"], c["hkv"], c["ps"], ctypes.c_float(1 / math.sqrt(c["d"])), 0, n_splits, stream]
    if scratch is not None:
        head.append(P(scratch))
    return getattr(lib, fn_name)(*head, *tail)


@pytest.mark.parametrize("d", [128, 64])
def test_static_scratch_entry_point_matches_the_ordinary_one(d):
    from simple_inference_b200 import ops
    lib = ops.attention_library(d)
    lib.si_attn_decode_scratch_floats.restype = ctypes.c_longlong
    calls = [
        (_case(3, [700, 64, 2047], 24, 8, d, 16, seed=1), 7),
        (_case(5, [10, 300, 1500, 0, 129], 8, 4, d, 8, seed=2), 4),   # smaller: old contents remain
    ]
    for c, splits in calls:
        need = lib.si_attn_decode_scratch_floats(c["n"], c["hq"], splits)
        assert 0 < need <= SCRATCH_FLOATS
        want = torch.zeros(c["n"], c["hq"] * d, device="cuda", dtype=torch.bfloat16)
        scratch = torch.empty(need, device="cuda", dtype=torch.float32)
        assert _call(lib, "si_attn_decode", c, want, splits, scratch) == 0
        got = torch.zeros_like(want)                # the caller still passes inputs and outputs
        held = torch.cuda.memory_allocated()
        assert _call(lib, "si_attn_decode_static", c, got, splits) == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == held   # no scratch came from torch either
        # same kernels, same split count, same order of sums: bit for bit
        assert torch.equal(got, want)
        # and against plain float32 attention over the same pages
        from tests import twin_ops
        ref = torch.zeros(c["n"], c["hq"] * d, device="cuda")
        twin_ops.attention_generic(c["q"].float(), c["pool"].float(), c["table"], c["single"],
                                   c["positions"], ref, c["hq"], c["hkv"], d, 1 / math.sqrt(d), None)
        assert (got.float() - ref).abs().max() < 2e-2


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from simple_inference_b200 import ops
    lib = ops.attention_library(128)
    lib.si_attn_decode_scratch_floats.restype = ctypes.c_longlong
    c = _case(16, [100] * 16, 24, 8, 128, 16, seed=3)
    assert lib.si_attn_decode_scratch_floats(16, 24, 32) > SCRATCH_FLOATS
    out = torch.full((16, 24 * 128), 5.0, device="cuda", dtype=torch.bfloat16)
    assert _call(lib, "si_attn_decode_static", c, out, 32) == -4     # SI_ERR_TOO_LARGE
    torch.cuda.synchronize()
    assert float(out.float().min()) == 5.0                           # nothing ran
    # absurd sizes are refused by their ranges, before any product of them is formed
    huge = dict(c, n=2**31 - 1, hq=65535)
    assert _call(lib, "si_attn_decode_static", huge, out, 65535) == -4
    assert _call(lib, "si_attn_decode_static", dict(c, hq=65536 * 8, hkv=8), out, 2) == -4
    assert _call(lib, "si_attn_decode_static", c, out, 70000) == -4
    torch.cuda.synchronize()
    assert float(out.float().min()) == 5.0
    assert _call(lib, "si_attn_decode_static", c, out, 2) == 0       # the same batch with fewer splits fits
    torch.cuda.synchronize()
    assert float(out.float().abs().max()) < 5.0
