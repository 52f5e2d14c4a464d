#!/usr/bin/env python3
"""The reference arm of ``bench.py``: the unmodified reference, timed on the same workload.

``baseline/_ref`` holds a byte-identical copy of the reference project (a flat
folder of importable modules; pip cannot install it because its
``pyproject.toml`` names no packages).  This script puts that folder first on
``sys.path`` and imports nothing of ``simple_inference_b200``.  It builds the
reference's own ``LlamaModel`` at the Llama 3.2 3B shape in bfloat16 with random
weights (the reference's tests fill parameters the same way,
``serving/test_paged_kv_cache.py:204-208``), hands it to the reference's own
``InferenceEngine`` with its stock Triton kernels and CUDA graphs
(``serving/engine.py:96-113``), lets the engine prefill ``batch`` prompts of
2,048 uniform-random ids and then times calls of its ``step()``: CUDA events
around the loop give ``value``, the wall clock gives ``e2e`` (a ``step()``
takes host token ids and returns host token ids, ``serving/engine.py:314-349``).
The steady-state loop follows ``benchmarks/bench_engine_cudagraph.py:60-112``,
except that requests advance as they do in serving instead of being reset.

Prints one JSON line with ``"impl": "reference"``; on any failure before the
headline number the line is ``{"impl": "reference", "unavailable": "<why>"}``.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time
import traceback
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF = HERE / "_ref"

MAX_CONTEXT = 4096
DECODE_CONTEXT = 2048
PREFILL_TOKENS = 2048
PAGE_SIZE = 16


def unavailable(why: str) -> int:
    print(json.dumps({"impl": "reference", "unavailable": " ".join(why.split())[:600]}))
    return 0


def build_model(torch):
    from config import ModelConfig
    from model.llama import LlamaModel
    cfg = ModelConfig.llama_3_2_3b()
    device = torch.device("cuda")
    with torch.device("cuda"):
        model = LlamaModel(cfg, device)
    model.to(device, torch.bfloat16)
    model.eval()
    gen = torch.Generator(device="cuda").manual_seed(0)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.dim() == 1:   # norm gains: 1 + N(0, 0.1), as in this repository's own arm
                p.copy_((1.0 + 0.1 * torch.randn(p.shape, generator=gen, device="cuda")).to(p.dtype))
            else:
                p.copy_((0.02 * torch.randn(p.shape, generator=gen, device="cuda")).to(p.dtype))
    return cfg, model


def steady_engine(torch, model, batch, new_tokens):
    """The reference engine with ``batch`` requests prefilled to DECODE_CONTEXT tokens."""
    from serving.engine import InferenceEngine
    from serving.request import RequestState
    eng = InferenceEngine(model=model, max_running=batch, max_seq_len=MAX_CONTEXT,
                          block_size=PAGE_SIZE, eos_id=-1, temperature=0.0, warmup=True,
                          use_cuda_graphs=True)
    g = torch.Generator().manual_seed(7)
    for _ in range(batch):
        ids = torch.randint(0, model.cfg.vocab_size, (DECODE_CONTEXT,), generator=g).tolist()
        eng.add_request(ids, new_tokens)
    for _ in range(batch + 4):
        eng.step()
        if sum(r.state is RequestState.DECODE for r in eng.scheduler.running) == batch:
            break
    else:
        raise RuntimeError("the reference engine did not bring every request to DECODE")
    return eng


def time_decode(torch, model, batch, steps, warmup, clocks=None):
    eng = steady_engine(torch, model, batch, steps + warmup + 8)
    for _ in range(warmup):
        assert len(eng.step()) == batch
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if clocks:
        clocks.mark_start()
    t0 = time.perf_counter()
    start.record()
    for _ in range(steps):
        out = eng.step()
        assert len(out) == batch
    end.record()
    torch.cuda.synchronize()
    wall_ms = (time.perf_counter() - t0) * 1e3 / steps
    if clocks:
        clocks.mark_end()
    dev_ms = start.elapsed_time(end) / steps
    info = {"backend": eng.decode_backend, "cuda_graphs_active": bool(eng.cuda_graphs_active)}
    # what its step copies: ids, positions and the whole block table as int64 host to
    # device (serving/paged_decoder.py:207-257), the sampled ids back
    bucket = eng.decoder.bucket_for(batch) or batch
    h2d = bucket * 8 * (2 + eng.decoder.max_blocks)
    d2h = batch * 8
    eng.reset()
    del eng
    torch.cuda.empty_cache()
    return dev_ms, wall_ms, h2d, d2h, info


def time_prefill(torch, model, reps=3):
    from serving.engine import InferenceEngine
    eng = InferenceEngine(model=model, max_running=1, max_seq_len=MAX_CONTEXT,
                          block_size=PAGE_SIZE, eos_id=-1, temperature=0.0, warmup=True,
                          use_cuda_graphs=True)
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, model.cfg.vocab_size, (PREFILL_TOKENS,), generator=g).tolist()
    times = []
    for _ in range(reps + 1):
        eng.reset()
        eng.add_request(ids, 4)
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        out = eng.step()     # admits, runs the whole prompt, draws the first token
        end.record()
        torch.cuda.synchronize()
        assert len(out) == 1
        times.append(start.elapsed_time(end))
    eng.reset()
    del eng
    torch.cuda.empty_cache()
    times = sorted(times[1:])
    return times[len(times) // 2]


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--no-points", action="store_true")
    args = ap.parse_args()
    warmup = max(args.warmup, 3)

    if not (REF / "serving" / "engine.py").is_file():
        return unavailable("baseline/_ref does not hold the reference (copy the reference project "
                           "there unchanged: cp -r <reference> baseline/_ref)")
    os.environ.setdefault("PYTHONDONTWRITEBYTECODE", "1")
    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    os.environ.setdefault("TRITON_CACHE_DIR", "/tmp/si_reference_triton_cache")
    sys.path[:] = [str(REF)] + [p for p in sys.path
                                if Path(p or ".").resolve() not in (HERE, HERE.parent)]
    try:
        import torch
        if not torch.cuda.is_available():
            return unavailable("no CUDA device")
        sys.path.append(str(HERE))
        from clock_sampler import ClockSampler
        cfg, model = build_model(torch)
        with ClockSampler() as clocks:
            dev_ms, wall_ms, h2d, d2h, info = time_decode(torch, model, args.batch, args.steps,
                                                          warmup, clocks)
        clock_record = clocks.summary()
    except Exception as e:  # the reference's own code failed: say how, verbatim
        tb = traceback.format_exc().strip().splitlines()
        return unavailable(f"the reference failed on this box: {type(e).__name__}: {e} "
                           f"[{tb[-3] if len(tb) > 2 else ''}]")

    line = {
        "metric": "decode tok/s, Llama 3.2 3B shape, batch 8, context 2048 (1 GPU)",
        "value": round(args.batch / (dev_ms * 1e-3), 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": warmup, "ms_per_step": round(dev_ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02) seed 0, uniform-random token ids",
        "impl": "reference",
        "config": {
            "model": "llama-3.2-3b-shape", "layers": cfg.num_hidden_layers,
            "layers_of_full_model": cfg.num_hidden_layers, "hidden": cfg.hidden_size,
            "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size,
            "vocab": cfg.vocab_size, "global_batch": args.batch, "seq_len": DECODE_CONTEXT,
            "max_context": MAX_CONTEXT, "page_size": PAGE_SIZE, "prefill_tokens": PREFILL_TOKENS,
            "parallelism": "single-gpu", "cuda_graph": info["cuda_graphs_active"],
            "backend": info["backend"],
            "l2": "inputs larger than L2: every step streams the weights (GBs) once",
        },
        "e2e": {"value": round(args.batch / (wall_ms * 1e-3), 1), "unit": "tokens/s",
                "ms_per_step": round(wall_ms, 4), "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h},
        "gpu_launches": 0,   # none of this repository's kernels run in this arm
        "clocks": clock_record,
    }
    errors = {}
    try:
        pre_ms = time_prefill(torch, model)
        line["prefill"] = {"value": round(PREFILL_TOKENS / (pre_ms * 1e-3), 1),
                           "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 3)}
    except Exception as e:
        errors["prefill"] = f"{type(e).__name__}: {e}"[:300]
    if not args.no_points:
        points = {}
        for b in (1, 64):
            try:
                pms, _, _, _, _ = time_decode(torch, model, b, max(10, args.steps // 2), warmup)
                points[f"decode_b{b}"] = round(b / (pms * 1e-3), 1)
            except Exception as e:
                errors[f"decode_b{b}"] = f"{type(e).__name__}: {e}"[:300]
                torch.cuda.empty_cache()
        line["points"] = points
    if errors:
        line["errors"] = errors
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
