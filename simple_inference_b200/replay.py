"""Trace replay: feeds given token ids through the model step by step, writes logits.

It samples nothing and has no forward pass, cache or loader of its own: it
loads the model as generation does (``load_model``), keeps a ``CacheManager``
sized for ``--max-tokens`` and drives ``ModelRunner.step``, the step function
that the engine uses.  Steps come from standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted, ``OUT/<step>.f32`` holds the logits at
the wanted places as little-endian float32 ``[wanted, vocab]``, in the order of
the entries and of ``want``.  After every step a line ``done <step>`` is printed
and flushed.  The reference has nothing like it; its closest relatives compare
greedy ids across batching regimes (``serving/test_engine.py:126-158``).
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import numpy as np
import torch

from . import ops
from .cache.manager import CacheManager
from .engine.batch import StepEntry
from .engine.runner import ModelRunner
from .models.load import load_model

PAGE_SIZE = 16          # tokens per page; request lengths are rounded up to 64, a multiple of it
MAX_LIVE_REQUESTS = 8   # the protocol promises at most four at a time
STEP_TOKEN_CAP = 4096   # a step that brings more tokens runs as several batches


def _split(entries: list[StepEntry], cap: int) -> list[list[StepEntry]]:
    """Cut a step into batches of at most ``cap`` tokens, keeping each request's order.

    A request appears at most once per batch, so a long portion is continued in
    the next batch; cutting does not change any logit beyond rounding.
    """
    pending = [(e.request, list(e.tokens), sorted(set(e.want)), 0) for e in entries]
    batches: list[list[StepEntry]] = []
    while pending:
        room, batch, rest = cap, [], []
        for req, toks, want, base in pending:
            if room == 0:
                rest.append((req, toks, want, base))
                continue
            n = min(len(toks), room)
            batch.append(StepEntry(req, toks[:n], [w - base for w in want if base <= w < base + n]))
            room -= n
            if n < len(toks):
                rest.append((req, toks[n:], want, base + n))
        batches.append(batch)
        pending = rest
    return batches


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at a time (each rounded up to 64)")
    args = ap.parse_args(argv)

    if not torch.cuda.is_available():
        print("trace_run: no CUDA device; the engine has no CPU path", file=sys.stderr)
        return 2
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)

    print(f"trace_run: loading {args.model} ({args.dtype})", file=sys.stderr, flush=True)
    cfg, model = load_model(args.model, args.dtype, "cuda")
    rt = model.rt
    num_pages = max(1, (args.max_tokens + PAGE_SIZE - 1) // PAGE_SIZE)
    max_seq_len = min(model.plan.max_positions, num_pages * PAGE_SIZE)
    cap = min(STEP_TOKEN_CAP, max_seq_len * MAX_LIVE_REQUESTS)
    cache = CacheManager(model.cache_specs(), PAGE_SIZE, num_pages, MAX_LIVE_REQUESTS, cap,
                         dtype=rt.dtype, device=rt.device)
    runner = ModelRunner(model, cache, rt, cap, MAX_LIVE_REQUESTS, max_seq_len,
                         cuda_graphs=(args.dtype == "bfloat16"), max_logit_rows=cap)
    vocab = model.plan.vocab_size

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            rid, toks = e["id"], [int(t) for t in e["tokens"]]
            if any(t < 0 or t >= vocab for t in toks):
                raise ValueError(f"step {step}: token id outside the vocabulary of {vocab}")
            if not cache.is_admitted(rid):
                cache.admit(rid, len(toks))
            else:
                cache.reserve_to(rid, cache.length(rid) + len(toks))
            entries.append(StepEntry(rid, toks, [int(w) for w in e.get("want", [])]))
        chunks: list[np.ndarray] = []
        if entries:
            # order of rows: entries in order, each entry's want in the order given
            order: list[tuple[int, int]] = []
            for i, e in enumerate(entries):
                order.extend((i, w) for w in e.want)
            got: dict[tuple[int, int], np.ndarray] = {}
            index_of = {e.request: i for i, e in enumerate(entries)}
            consumed = {e.request: 0 for e in entries}
            for batch in _split(entries, cap):
                logits = runner.step(batch)
                host = logits.cpu().numpy() if logits.shape[0] else None
                ops.check_status(rt.device)
                r = 0
                for b in batch:
                    base = consumed[b.request]
                    for w in b.want:
                        got[(index_of[b.request], base + w)] = host[r]
                        r += 1
                    consumed[b.request] = base + len(b.tokens)
            chunks = [got[key] for key in order]
        if chunks:
            arr = np.ascontiguousarray(np.stack(chunks), dtype="<f4")
            arr.tofile(out_dir / f"{step}.f32")
        for rid in rec.get("end", []):
            if cache.is_admitted(rid):
                cache.release(rid)
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
