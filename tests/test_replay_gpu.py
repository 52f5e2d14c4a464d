"""Trace replay on the GPU against the plain model: every way of cutting the work.

The same requests are replayed whole, with the last 32 tokens one by one, in
portions of changing size down to two tokens, and mixed with other requests in
a pool so small that pages are used again; in float32 and in bfloat16.  Every
logit row that trace_run writes is compared with the plain whole-sequence model.
"""

import pytest
import torch
from safetensors.torch import load_file, save_file

from simple_inference_b200.weights import write_random_model
from tests import plain_llama
from tests.conftest import TINY, random_ids
from tests.replay_util import Trace

pytestmark = pytest.mark.gpu

# Tolerances on logits whose standard deviation is 0.2 to 0.3: float32 differs from the plain
# model by summation order only; bfloat16 by the rounding of activations, measured at up to
# 7.5e-3 over all configurations and cuts but the sharpened Tiny D, and allowed twice that.
# One key and value taken from a wrong token in one layer moves these logits by 0.019 to 0.9
# (tests/test_plain.py proves it on the CPU), so it cannot hide under the bound.
TOL = {"float32": 2e-5, "bfloat16": 1.5e-2}
# Sharpened Tiny D: scores 36 times larger make the softmax of its 128-wide heads feel every
# rounding of q and k (measured 0.053 to 0.062); a wrong key moves its logits by 0.34 and more.
TOL_SHARP_D = {"float32": 2e-5, "bfloat16": 0.15}
# between two ways of cutting the same request in the same dtype
CUT_TOL = {"float32": 2e-6, "bfloat16": 1.5e-2}


@pytest.fixture(scope="module")
def cases(model_folders, tmp_path_factory):
    """name -> (folder, plain config, plain weights, sequences, plain logits per sequence)."""
    folders = dict(model_folders)
    # "sharp": Tiny B with queries and keys scaled up, so that each row of attention rests on
    # a few keys; a key read from a wrong page or position then changes the logits visibly.
    sharp = tmp_path_factory.mktemp("tiny_sharp")
    write_random_model(sharp, TINY["B"], seed=21)
    t = load_file(str(sharp / "model.safetensors"))
    for k in list(t):
        if "q_proj" in k or "k_proj" in k:
            t[k] = (t[k].float() * 6.0).to(t[k].dtype)
    save_file(t, str(sharp / "model.safetensors"))
    folders["sharp"] = sharp
    # the same for Tiny D, whose head size of 128 and long prompts take the tcgen05 attention,
    # the TMA-fed decode attention and the tcgen05 products
    sharp_d = tmp_path_factory.mktemp("tiny_sharp_d")
    write_random_model(sharp_d, TINY["D"], seed=23)
    t = load_file(str(sharp_d / "model.safetensors"))
    for k in list(t):
        if "q_proj" in k or "k_proj" in k:
            t[k] = (t[k].float() * 6.0).to(t[k].dtype)
    save_file(t, str(sharp_d / "model.safetensors"))
    folders["sharpD"] = sharp_d
    out = {}
    for name, folder in folders.items():
        cfg, w = plain_llama.read_folder(folder)
        top = min(cfg["max_position_embeddings"], 420 if name in LONG else 230)
        lens = [top, 97, 64, 33, 5, 150][: 6 if top > 128 else 5]
        lens = [min(n, top) for n in lens]
        seqs = [random_ids(n, cfg["vocab_size"], 100 + i) for i, n in enumerate(lens)]
        out[name] = (folder, cfg, w, seqs, [plain_llama.forward(cfg, w, s) for s in seqs])
    return out


LONG = ("D", "sharpD", "E")   # head sizes of the Blackwell kernels: prompts long enough to reach them


def _tol(table, dtype, what):
    return TOL_SHARP_D[dtype] if what.startswith("sharpD") else table[dtype]


def _check(got, want, dtype, what):
    diff = (got - want).abs().max().item()
    print(f"max |engine - plain| {dtype} {what}: {diff:.2e}")     # shown by pytest -rA
    assert diff < _tol(TOL, dtype, what), f"{what}: max |engine - plain| = {diff}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "sharp", "sharpD"])
def test_whole_then_last_32_then_portions(name, dtype, cases, tmp_path):
    folder, cfg, w, seqs, plain = cases[name]
    with Trace(folder, dtype, tmp_path, max_tokens=512 if name in LONG else 256) as tr:
        for i, (ids, ref) in enumerate(zip(seqs[:3], plain[:3])):
            n = len(ids)
            # (1) alone and whole, every position wanted
            whole = tr.step([(f"w{i}", ids, range(n))], end=[f"w{i}"])
            _check(whole, ref, dtype, f"{name} seq {i} whole")
            # (2) most of it in one step, the last 32 tokens one by one
            head = n - 32
            rows = [tr.step([(f"d{i}", ids[:head], [head - 1])])]
            for p in range(head, n):
                rows.append(tr.step([(f"d{i}", [ids[p]], [0])], end=[f"d{i}"] if p == n - 1 else []))
            tail = torch.cat(rows)
            _check(tail, ref[head - 1:], dtype, f"{name} seq {i} last 32 one by one")
            assert (tail - whole[head - 1:]).abs().max() < _tol(CUT_TOL, dtype, name)
            # (3) portions of changing size, down to two tokens
            sizes, p, rows = [7, 2, 13, 3, 2, 31, 2, 5, 64, 2, 9], 0, []
            k = 0
            while p < n:
                c = min(sizes[k % len(sizes)], n - p)
                rows.append(tr.step([(f"p{i}", ids[p:p + c], range(c))],
                                    end=[f"p{i}"] if p + c == n else []))
                p += c
                k += 1
            parts = torch.cat(rows)
            _check(parts, ref, dtype, f"{name} seq {i} in portions")
            assert (parts - whole).abs().max() < _tol(CUT_TOL, dtype, name)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "sharp", "D", "E", "sharpD"])
def test_mixed_batches_with_pages_used_again(name, dtype, cases, tmp_path):
    """Up to four live requests, portions of some beside decoded tokens of others, in a pool
    of 320 tokens (20 pages) that the requests need 2.5 times over.  The configurations with
    heads of 128 get longer prompts, a pool of 640 tokens that they need 1.5 times over, and
    portions of 64, 128 and 200 tokens, so that the tcgen05 attention and products run beside
    decoded tokens of other requests while pages change hands."""
    folder, cfg, w, seqs, plain = cases[name]
    lens = [len(s) for s in seqs]
    pool = 640 if name in LONG else 320
    assert sum((n + 63) // 64 * 64 for n in lens) > pool     # more than the pool: pages come back
    # each request: a prompt part fed in portions, then the rest token by token
    plan = {i: {"prompt": max(2, n - 20 - 3 * i), "fed": 0} for i, n in enumerate(lens)}
    portion = [9, 2, 200, 5, 128, 2, 64] if name in LONG else [9, 2, 30, 5, 17, 2, 64]
    waiting = list(range(len(seqs)))
    live: list[int] = []
    got = {i: {} for i in range(len(seqs))}
    with Trace(folder, dtype, tmp_path, max_tokens=pool) as tr:
        k = 0
        while waiting or live:
            # admit while at most four are live and the rounded-up lengths fit in the pool
            while waiting and len(live) < 4 and \
                    sum((lens[j] + 63) // 64 * 64 for j in live + [waiting[0]]) <= pool:
                live.append(waiting.pop(0))
            entries, ending, index = [], [], []
            for i in live:
                st, ids = plan[i], seqs[i]
                if st["fed"] < st["prompt"]:
                    c = min(portion[k % len(portion)], st["prompt"] - st["fed"])
                    if st["prompt"] - st["fed"] - c == 1:   # never leave a portion of one token
                        c += 1
                    k += 1
                else:
                    c = 1
                if (k + i) % 5 == 0 and c == 1 and len(live) > 1:
                    continue                                 # a request may sit a step out
                want = list(range(c))
                entries.append((f"r{i}", ids[st["fed"]:st["fed"] + c], want))
                index.append((i, st["fed"], c))
                st["fed"] += c
                if st["fed"] == len(ids):
                    ending.append(i)
            k += 1
            if not entries:
                continue
            rows = tr.step(entries, end=[f"r{i}" for i in ending])
            r = 0
            for i, start, c in index:
                for q in range(c):
                    got[i][start + q] = rows[r]
                    r += 1
            live = [i for i in live if i not in ending]
    for i, ref in enumerate(plain):
        mine = torch.stack([got[i][p] for p in range(len(seqs[i]))])
        _check(mine, ref, dtype, f"{name} request {i} in mixed batches")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(dtype, cases, tmp_path):
    folder, cfg, w, seqs, plain = cases["B"]
    ids, ref = seqs[0], plain[0]
    with Trace(folder, dtype, tmp_path, max_tokens=512) as tr:
        # the first tokens of a sequence, one by one from position 0, beside a second request
        rows = []
        other, oref = seqs[1], plain[1]
        orow = []
        for p in range(len(ids)):
            entries = [("long", [ids[p]], [0])]
            if p < len(other):
                entries.append(("other", [other[p]], [0]))
            out = tr.step(entries)
            rows.append(out[0])
            if p < len(other):
                orow.append(out[1])
        _check(torch.stack(rows), ref, dtype, "decoding token by token from the first token")
        _check(torch.stack(orow), oref, dtype, "second request decoded beside it")
        # nothing wanted: no file, the cache still advances
        assert tr.step([("quiet", seqs[2][:10], [])]) is None
        out = tr.step([("quiet", seqs[2][10:12], [1])])
        _check(out, plain[2][11:12], dtype, "after a step that wanted nothing")
