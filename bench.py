#!/usr/bin/env python3
"""Headline benchmark: decode tokens/s of the Llama 3.2 3B shape on one B200.

Contract: ``python bench.py --gpus N --steps K --warmup W`` prints ONE JSON line.
A step is one decode step of a batch of 8 requests at context 2,048 (the decode
workload of the reference's headline configuration), bfloat16, random weights,
synthetic token ids.  ``value`` is decoded tokens per second timed on the device
with CUDA events; ``e2e`` is the same through ``InferenceEngine.step()`` with
host token ids in and sampled ids out every step.  The line also carries the
prefill of 2,048 tokens, the decode roofline (weights + live cache bytes over
the step time against the measured copy bandwidth) and decode at batch 1 and 64.
This engine runs on one GPU: for N > 1 it says so and exits with 2.

``--impl reference`` runs the unmodified reference from ``baseline/_ref`` on the
same workload through its own engine (``baseline/reference_arm.py``, a process
of its own) and prints the same line with ``"impl": "reference"``.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

LLAMA_3_2_3B = {
    "architectures": ["LlamaForCausalLM"],
    "num_hidden_layers": 28, "hidden_size": 3072, "num_attention_heads": 24,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 8192, "vocab_size": 128256,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 131072,
    "torch_dtype": "bfloat16",
}
MAX_CONTEXT = 4096
DECODE_CONTEXT = 2048
PREFILL_TOKENS = 2048
PAGE_SIZE = 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            raw = json.loads(path.read_text())
            out = dict(FALLBACK_PEAKS)
            for k in out:
                if isinstance(raw.get(k), (int, float)):
                    out[k] = float(raw[k])
            return out, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


from baseline.clock_sampler import ClockSampler  # noqa: E402


def matmul_params(cfg) -> tuple[int, int]:
    """(elements of the layers' matrices, elements of the output head)."""
    h, d = cfg.hidden_size, cfg.head_dim
    per_layer = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * d * h \
        + h * cfg.num_attention_heads * d + 3 * h * cfg.intermediate_size
    return per_layer * cfg.num_hidden_layers, cfg.vocab_size * h


def kv_bytes_per_token(cfg, elt=2) -> int:
    return 2 * cfg.num_key_value_heads * cfg.head_dim * elt * cfg.num_hidden_layers


EAGER = False  # --eager: no CUDA graphs, so that a profiler sees every kernel as its own launch


def build_runner(model, batch, layers_note=None):
    import torch
    from simple_inference_b200.cache import CacheManager, pages_for
    from simple_inference_b200.engine import ModelRunner
    rt = model.rt
    pages = batch * pages_for(MAX_CONTEXT, PAGE_SIZE)
    cache = CacheManager(model.cache_specs(), PAGE_SIZE, pages, batch, max(PREFILL_TOKENS, batch),
                         dtype=rt.dtype, device=rt.device)
    runner = ModelRunner(model, cache, rt, max(PREFILL_TOKENS, batch), batch, MAX_CONTEXT,
                         cuda_graphs=not EAGER)
    return cache, runner


def fill_context(cache, runner, batch, vocab, seed):
    """Admit ``batch`` requests and run their first DECODE_CONTEXT - 1 tokens."""
    import torch
    from simple_inference_b200.engine import StepEntry
    g = torch.Generator().manual_seed(seed)
    for b in range(batch):
        cache.admit(b, MAX_CONTEXT)
        ids = torch.randint(0, vocab, (DECODE_CONTEXT - 1,), generator=g).tolist()
        for i in range(0, len(ids), runner.max_step_tokens):   # in portions the runner takes
            runner.step([StepEntry(b, ids[i:i + runner.max_step_tokens], [])])
    torch.cuda.synchronize()


def time_decode(model, cfg, batch, steps, warmup, sample_clocks=False):
    """Device-timed decode: per step one metadata copy, the captured graph, the sampling kernel."""
    import torch
    from simple_inference_b200 import ops
    from simple_inference_b200.engine import StepEntry
    from simple_inference_b200.sampling import Sampler, SamplingParams
    cache, runner = build_runner(model, batch)
    fill_context(cache, runner, batch, cfg.vocab_size, seed=batch)
    sampler = Sampler(model.rt.device, batch)
    g = torch.Generator().manual_seed(1000 + batch)
    feed = torch.randint(0, cfg.vocab_size, (steps + warmup, batch), generator=g).tolist()
    greedy = [(SamplingParams(), 0, 0)] * batch

    def one(i):
        logits = runner.step([StepEntry(b, [feed[i][b]], [0]) for b in range(batch)])
        sampler.sample_on_device(logits)  # no read-back inside the device-timed region

    sampler.sample(runner.step([StepEntry(b, [1], [0]) for b in range(batch)]), greedy)  # sets params
    clocks = ClockSampler() if sample_clocks else None
    if clocks:
        clocks.__enter__()
    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    k0, r0 = ops.launch_count, runner.replayed_kernels
    torch.cuda.synchronize()
    if clocks:
        clocks.mark_start()
    torch.cuda.profiler.start()  # a profiler started with --profile-from-start off sees only this
    start.record()
    for i in range(warmup, warmup + steps):
        one(i)
    end.record()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    if clocks:
        clocks.mark_end()
        clocks.__exit__(None, None, None)
    ms = start.elapsed_time(end) / steps
    launches = (ops.launch_count - k0) + (runner.replayed_kernels - r0)
    ctx_mean = DECODE_CONTEXT + 1 + warmup + (steps - 1) / 2
    check = check_against_eager(runner, cache, batch, feed[0]) if not EAGER else None
    del runner, cache
    torch.cuda.empty_cache()
    return ms, launches, ctx_mean, (clocks.summary() if clocks else None), check


def time_products(cfg, batch):
    """The matrix products of a decode step, each on its own: 28 copies of one layer's matrix (so
    that every launch streams its weights from memory) run back to back from a CUDA graph, as
    they follow each other in a step; microseconds per product and the rate at which it streams
    its weights.  Kernels timed alone under a profiler cannot show what the prefetch before the
    wait on the preceding kernel gains; this can."""
    import torch
    from simple_inference_b200 import ops
    from simple_inference_b200.engine.batch import Workspace
    dev = torch.device("cuda:0")
    h, d = cfg.hidden_size, cfg.head_dim
    qkv_rows = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * d
    shapes = [("qkv", qkv_rows, h, "plain"), ("o", h, cfg.num_attention_heads * d, "residual"),
              ("gate_up", cfg.intermediate_size, h, "swiglu"), ("down", h, cfg.intermediate_size, "residual"),
              ("head", cfg.vocab_size, h, "logits")]
    ws = Workspace(dev, max(batch, 16))
    out = {"batch": batch}
    for name, n, k, kind in shapes:
        rows = 2 * n if kind == "swiglu" else n
        copies = 4 if kind == "logits" else cfg.num_hidden_layers
        mats = [torch.randn(rows, k, device=dev).bfloat16() * 0.02 for _ in range(copies)]
        x = torch.randn(batch, k, device=dev).bfloat16()
        y = torch.empty(batch, n, device=dev, dtype=torch.float32 if kind == "logits" else torch.bfloat16)

        y2 = torch.empty(batch, rows, device=dev, dtype=torch.bfloat16) if kind == "swiglu" else None

        def run(w):
            if kind == "swiglu" and ops.can_fuse_swiglu(x, w):
                ops.linear_swiglu(x, w, y)
            elif kind == "swiglu":   # between the two fused kernels: the product, then the activation
                ops.linear(x, w, y2)
                ops.swiglu(y2, y)
            elif kind == "residual":
                ops.linear_for_residual(x, w, ws, "bench", True)
            else:
                ops.linear(x, w[:n], y)
        for w in mats:
            run(w)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(3):
                for w in mats:
                    run(w)
        g.replay()
        torch.cuda.synchronize()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        g.replay()
        g.replay()
        s1.record()
        torch.cuda.synchronize()
        us = s0.elapsed_time(s1) * 1e3 / (6 * copies)
        out[name] = {"rows": rows, "k": k, "us": round(us, 2), "gb_s": round(rows * k * 2 / us / 1e3, 1)}
        del mats
        torch.cuda.empty_cache()
    return out


def decode_timeline(model, cfg, batch):
    """One decode step replayed from its CUDA graph under the kineto tracer: for every kernel its
    start, its duration and the time to the next kernel's start.  Under programmatic dependent
    launch kernels overlap (a kernel starts while its predecessor drains and waits inside), so
    the start-to-start column, not the durations, adds up to the step."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    from simple_inference_b200.engine import StepEntry
    cache, runner = build_runner(model, batch)
    fill_context(cache, runner, batch, cfg.vocab_size, seed=batch)

    def one(i):
        runner.step([StepEntry(b, [(i * 7 + b) % 1000], [0]) for b in range(batch)])
    for i in range(5):
        one(i)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for i in range(3):
            one(10 + i)
        torch.cuda.synchronize()
    ev = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA
          and "memcpy" not in e.name.lower() and "memset" not in e.name.lower()]
    ev.sort(key=lambda e: e.time_range.start)
    ev = ev[-(len(ev) // 3):]   # the last of the three steps
    t0, total = ev[0].time_range.start, ev[-1].time_range.end - ev[0].time_range.start
    rows = [(e.name.split("(")[0].replace("void ", "").replace("si::", "")[:48],
             e.time_range.start - t0, e.time_range.end - e.time_range.start) for e in ev]
    lines = [f"decode step, batch {batch}, context {DECODE_CONTEXT}, {cfg.num_hidden_layers} layers: "
             f"{len(rows)} kernels, {total:.1f} us from the first kernel's start to the last one's end",
             "by kernel: share of the step (start to next start), launches, mean duration, mean start-to-start"]
    agg = {}
    for i, (name, start, dur) in enumerate(rows):
        nxt = rows[i + 1][1] if i + 1 < len(rows) else total
        a = agg.setdefault(name, [0, 0.0, 0.0])
        a[0] += 1; a[1] += dur; a[2] += nxt - start
    for name, (n, dur, wall) in sorted(agg.items(), key=lambda kv: -kv[1][2]):
        lines.append(f"  {100 * wall / total:5.1f} %  n={n:3d}  dur {dur / n:7.2f} us  start-to-start {wall / n:7.2f} us  {name}")
    k = len(rows) // 2
    while k < len(rows) - 10 and "rmsnorm" not in rows[k][0]:
        k += 1
    lines.append("one layer from the middle of the step: start (us), duration (us), kernel")
    for name, start, dur in rows[k:k + 9]:
        lines.append(f"  {start:9.2f}  {dur:7.2f}  {name}")
    del runner, cache
    torch.cuda.empty_cache()
    return "\n".join(lines)


def check_against_eager(runner, cache, batch, tokens):
    """Outside the timed region: one more step replayed from the graph, then the same tokens at
    the same positions run eagerly (their keys and values land in the same slots again), and the
    two sets of logits compared, as the reference's benchmark compares its decode backends
    (``benchmarks/bench_paged_cudagraph.py:239-261``).  A graph that replayed stale sizes or
    addresses would show here."""
    import torch
    from simple_inference_b200.engine import StepEntry
    entries = [StepEntry(b, [tokens[b]], [0]) for b in range(batch)]
    replayed = runner.step(entries).clone()
    starts = [cache.length(b) - 1 for b in range(batch)]
    ctx = runner.builder.build(entries, starts, runner.ws)
    eager = runner.model.forward(ctx, runner.layer_caches)
    torch.cuda.synchronize()
    diff = float((replayed - eager).abs().max())
    agree = float((replayed.argmax(-1) == eager.argmax(-1)).float().mean())
    spread = float(eager.std())
    ok = bool(torch.isfinite(replayed).all()) and diff < 0.25 * spread and agree >= 0.75
    return {"max_abs_logit_diff": round(diff, 5), "top1_agree": round(agree, 4),
            "logit_std": round(spread, 4), "ok": ok}


def time_e2e(model, cfg, batch, steps, warmup):
    """The same decode through InferenceEngine.step(): host ids in, sampled ids out, every step."""
    import torch
    from simple_inference_b200 import InferenceEngine
    eng = InferenceEngine(model, max_running=batch, max_seq_len=MAX_CONTEXT, block_size=PAGE_SIZE,
                          eos_id=-1, temperature=0.0, max_tokens_per_step=PREFILL_TOKENS,
                          use_cuda_graphs=True, warmup=False)
    g = torch.Generator().manual_seed(7)
    for _ in range(batch):
        eng.add_request(torch.randint(0, cfg.vocab_size, (DECODE_CONTEXT,), generator=g).tolist(),
                        steps + warmup + 4 * batch + 16)  # earlier requests decode while later ones prefill
    while any(r.prefilled < r.prompt_len for r in eng.scheduler.running) or eng.scheduler.waiting:
        eng.step()
    for _ in range(warmup):
        eng.step()
    torch.cuda.synchronize()
    sent0 = eng.runner.builder.words_sent
    t0 = time.perf_counter()
    for _ in range(steps):
        out = eng.step()
        assert len(out) == batch
    torch.cuda.synchronize()
    dt = (time.perf_counter() - t0) / steps
    # the step's description (counted by the builder as it copies) and the sampling options
    h2d = (eng.runner.builder.words_sent - sent0) * 4 // steps + eng.sampler.host_bytes
    d2h = batch * 4
    eng.reset()
    del eng
    torch.cuda.empty_cache()
    return dt * 1e3, h2d, d2h


def time_prefill(model, cfg, reps=5):
    import torch
    from simple_inference_b200.engine import StepEntry
    cache, runner = build_runner(model, 1)
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, cfg.vocab_size, (PREFILL_TOKENS,), generator=g).tolist()
    times = []
    for i in range(reps + 2):
        cache.admit(i, MAX_CONTEXT)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        if i == reps + 1:
            torch.cuda.profiler.start()
        start.record()
        runner.step([StepEntry(i, ids, [PREFILL_TOKENS - 1])])
        end.record()
        torch.cuda.synchronize()
        if i == reps + 1:
            torch.cuda.profiler.stop()
        times.append(start.elapsed_time(end))
        cache.release(i)
    del runner, cache
    torch.cuda.empty_cache()
    return sorted(times[2:])[len(times[2:]) // 2]


LLAMA_3_2_1B = dict(LLAMA_3_2_3B, num_hidden_layers=16, hidden_size=2048, num_attention_heads=32,
                    num_key_value_heads=8, head_dim=64, intermediate_size=8192)
LLAMA_3_1_8B = dict(LLAMA_3_2_3B, num_hidden_layers=32, hidden_size=4096, num_attention_heads=32,
                    num_key_value_heads=8, head_dim=128, intermediate_size=14336,
                    tie_word_embeddings=False,
                    rope_scaling=dict(LLAMA_3_2_3B["rope_scaling"], factor=8.0))


def workload_1b_continuous_batching(pk):
    """The reference's continuous-batching workload at the Llama 3.2 1B shape: 64 requests, prompt
    lengths uniform in 128..2048 (seeded), 256 output tokens each, all queued at once and run
    through ``InferenceEngine.step()`` until done (random weights, greedy, no stop token)."""
    import torch
    from simple_inference_b200 import InferenceEngine
    from simple_inference_b200.engine import RequestState
    from simple_inference_b200.models.load import random_model
    cfg, model = random_model(dict(LLAMA_3_2_1B), seed=1, dtype="bfloat16", device="cuda:0")
    n_req, n_out = 64, 256
    g = torch.Generator().manual_seed(11)
    lens = torch.randint(128, 2049, (n_req,), generator=g).tolist()
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    eng = InferenceEngine(model, max_running=n_req, max_seq_len=2048 + n_out, block_size=PAGE_SIZE,
                          eos_id=-1, temperature=0.0, max_tokens_per_step=2048, warmup=True)
    reqs = [eng.add_request(p, n_out) for p in prompts]
    layer_params, head_params = matmul_params(cfg)
    weight_bytes = 2 * (layer_params + head_params)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    steps = decode_steps = 0
    decode_s = decode_bytes = 0.0
    while eng.has_work():
        running = eng.scheduler.running
        all_decoding = (not eng.scheduler.waiting and len(running) == n_req and
                        all(r.state is RequestState.DECODE for r in running))
        live = sum(r.pos + 1 for r in running) if all_decoding else 0
        t1 = time.perf_counter()
        eng.step()
        if all_decoding:   # a step of 64 decoded tokens and nothing else (the sampled ids came home)
            decode_s += time.perf_counter() - t1
            decode_bytes += weight_bytes + live * kv_bytes_per_token(cfg)
            decode_steps += 1
        steps += 1
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    assert all(len(r.generated) == n_out for r in reqs)
    out = {
        "model": "llama-3.2-1b-shape", "layers": cfg.num_hidden_layers, "hidden": cfg.hidden_size,
        "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
        "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
        "requests": n_req, "prompt_tokens": sum(lens), "output_tokens": n_req * n_out,
        "wall_s": round(wall, 3), "engine_steps": steps,
        "output_tok_s": round(n_req * n_out / wall, 1),
        "total_tok_s": round((sum(lens) + n_req * n_out) / wall, 1),
    }
    if decode_steps:
        achieved = decode_bytes / decode_s / 1e9
        out["decode_b64"] = {"steps": decode_steps, "ms_per_step": round(decode_s / decode_steps * 1e3, 4),
                             "tok_s": round(n_req * decode_steps / decode_s, 1),
                             "roofline_frac": round(achieved / pk["hbm_gbs"], 4), "gb_s": round(achieved, 1)}
    eng.reset()
    del eng, model
    torch.cuda.empty_cache()
    return out


def workload_8b_long_context(pk):
    """The long-context workload at the Llama 3.1 8B shape: 16 prompts of 8,192 ids run in portions
    of 2,048 tokens, then decoding at batch 16 over 17 GB of cache, through ``InferenceEngine.step()``."""
    import torch
    from simple_inference_b200 import InferenceEngine
    from simple_inference_b200.engine import RequestState
    from simple_inference_b200.models.load import random_model
    cfg, model = random_model(dict(LLAMA_3_1_8B), seed=2, dtype="bfloat16", device="cuda:0")
    n_req, n_prompt, n_out = 16, 8192, 48
    g = torch.Generator().manual_seed(12)
    prompts = [torch.randint(0, cfg.vocab_size, (n_prompt,), generator=g).tolist() for _ in range(n_req)]
    eng = InferenceEngine(model, max_running=n_req, max_seq_len=n_prompt + 2 * n_out + n_req * 4,
                          block_size=PAGE_SIZE, eos_id=-1, temperature=0.0, max_tokens_per_step=2048 + n_req,
                          chunk_size=2048, warmup=True)
    for p in prompts:   # earlier requests decode while later ones are still being read
        eng.add_request(p, n_out + 4 * n_req)
    layer_params, head_params = matmul_params(cfg)
    weight_bytes = 2 * (layer_params + head_params)   # untied: the head is streamed, embedding rows are gathered
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    prefill_steps = 0
    while eng.scheduler.waiting or any(r.state is RequestState.PREFILL for r in eng.scheduler.running) \
            or not eng.scheduler.running:
        eng.step()
        prefill_steps += 1
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t0
    T, d = n_prompt, cfg.head_dim
    flops_per_prompt = 2 * T * layer_params + 2 * head_params \
        + cfg.num_hidden_layers * 2 * cfg.num_attention_heads * d * T * (T + 1)
    for _ in range(3):
        eng.step()
    torch.cuda.synchronize()
    steps, live_sum = 20, 0
    t1 = time.perf_counter()
    for _ in range(steps):
        live_sum += sum(r.pos + 1 for r in eng.scheduler.running)
        assert len(eng.step()) == n_req
    torch.cuda.synchronize()
    decode_s = time.perf_counter() - t1
    step_bytes = weight_bytes + live_sum / steps * kv_bytes_per_token(cfg)
    achieved = step_bytes / (decode_s / steps) / 1e9
    out = {
        "model": "llama-3.1-8b-shape", "layers": cfg.num_hidden_layers, "hidden": cfg.hidden_size,
        "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
        "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
        "tied": False, "requests": n_req, "prompt_tokens_each": n_prompt, "portion": 2048,
        "prefill": {"tok_s": round(n_req * n_prompt / prefill_s, 1), "s": round(prefill_s, 3),
                    "engine_steps": prefill_steps,
                    "frac_of_sustained_peak": round(n_req * flops_per_prompt / prefill_s /
                                                    (pk["bf16_tflops_sustained"] * 1e12), 4),
                    "note": "earlier requests decode beside the later prompts' portions"},
        "decode_b16": {"tok_s": round(n_req * steps / decode_s, 1),
                       "ms_per_step": round(decode_s / steps * 1e3, 4),
                       "mean_context": round(live_sum / steps / n_req, 1),
                       "gb_per_step": round(step_bytes / 1e9, 2), "gb_s": round(achieved, 1),
                       "roofline_frac": round(achieved / pk["hbm_gbs"], 4)},
    }
    eng.reset()
    del eng, model
    torch.cuda.empty_cache()
    return out


def run_reference(args) -> int:
    """Run ``baseline/reference_arm.py`` in a process of its own (so that nothing of this
    package is imported beside the reference) and pass its JSON line on."""
    cmd = [sys.executable, str(ROOT / "baseline" / "reference_arm.py"), "--steps", str(args.steps),
           "--warmup", str(args.warmup), "--batch", str(args.batch)]
    if args.no_points:
        cmd.append("--no-points")
    env = dict(os.environ)
    env.pop("PYTHONPATH", None)
    try:
        proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True,
                              env=env, cwd=str(ROOT / "baseline"), timeout=1500)
    except subprocess.TimeoutExpired:
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference arm did not finish within 25 minutes"}))
        return 0
    lines = [ln for ln in proc.stdout.splitlines() if ln.startswith("{")]
    if lines:
        print(lines[-1])
        return 0
    tail = " ".join(proc.stderr.strip().splitlines()[-3:])[:500]
    print(json.dumps({"impl": "reference", "unavailable":
                      f"the reference arm exited with {proc.returncode}: {tail}"}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers (named in config)")
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    ap.add_argument("--no-workloads", action="store_true",
                    help="skip the 1B continuous-batching and 8B long-context workloads")
    ap.add_argument("--only", choices=["decode", "prefill", "products"],
                    help="run one part and print a short record (for profiling; not the contract line)")
    ap.add_argument("--eager", action="store_true", help="no CUDA graphs (for kernel-level profiles)")
    ap.add_argument("--timeline", action="store_true",
                    help="with --only decode: the kernels of one replayed step with their real start "
                         "times (kineto), as text")
    ap.add_argument("--shape", choices=["3b", "1b", "8b"], default="3b",
                    help="with --only: the layer sizes (Llama 3.2 3B, 3.2 1B or 3.1 8B)")
    ap.add_argument("--context", type=int, default=None,
                    help="with --only decode: tokens each request holds (default 2048)")
    ap.add_argument("--prefill-tokens", type=int, default=None,
                    help="with --only prefill: length of the prompt (default 2048)")
    args = ap.parse_args()
    global EAGER, DECODE_CONTEXT, PREFILL_TOKENS, MAX_CONTEXT
    EAGER = args.eager
    if args.only and (args.context or args.prefill_tokens):   # other sizes than the headline's
        DECODE_CONTEXT = args.context or DECODE_CONTEXT
        PREFILL_TOKENS = args.prefill_tokens or PREFILL_TOKENS
        MAX_CONTEXT = max(MAX_CONTEXT, DECODE_CONTEXT + 2048, PREFILL_TOKENS)

    if args.impl == "reference":
        if args.gpus != 1:
            print(json.dumps({"impl": "reference", "unavailable":
                              "the reference engine runs on one GPU"}))
            return 0
        return run_reference(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not built")
        return 2
    warmup = max(args.warmup, 3)

    import torch
    from simple_inference_b200.models.load import random_model
    if not torch.cuda.is_available():
        print("bench.py: no CUDA device")
        return 1
    pk, pk_src = peaks()
    config = dict(LLAMA_3_2_3B)
    if args.only and args.shape != "3b":
        config = dict(LLAMA_3_2_1B if args.shape == "1b" else LLAMA_3_1_8B)
    full_layers = config["num_hidden_layers"]
    if args.layers:
        config["num_hidden_layers"] = args.layers
    if args.only == "products":
        from simple_inference_b200.config.registry import architecture_of
        cfg = architecture_of(config).config_class.from_dict(config)
        print(json.dumps(time_products(cfg, args.batch)))
        return 0
    cfg, model = random_model(config, seed=0, dtype="bfloat16", device="cuda:0")
    layer_params, head_params = matmul_params(cfg)
    weight_bytes = 2 * (layer_params + head_params)

    if args.only == "decode" and args.timeline:
        print(decode_timeline(model, cfg, args.batch))
        return 0
    if args.only == "decode":
        ms, launches, _, _, _ = time_decode(model, cfg, args.batch, args.steps, args.warmup)
        print(json.dumps({"only": "decode", "batch": args.batch, "context": DECODE_CONTEXT,
                          "layers": cfg.num_hidden_layers, "eager": EAGER,
                          "ms_per_step": round(ms, 4), "launches": launches}))
        return 0
    if args.only == "prefill":
        pre_ms = time_prefill(model, cfg, reps=max(1, args.steps))
        print(json.dumps({"only": "prefill", "tokens": PREFILL_TOKENS,
                          "layers": cfg.num_hidden_layers, "ms": round(pre_ms, 3)}))
        return 0

    # the prefill is one step of some 12 ms, timed alone like the burst product its fraction is taken
    # of: it runs before the seconds of decoding that bring the GPU to its power cap
    pre_ms = time_prefill(model, cfg)
    ms, launches, ctx_mean, clocks, check = time_decode(model, cfg, args.batch, args.steps, warmup, True)
    graph_check = {f"b{args.batch}": check}
    step_bytes = weight_bytes + args.batch * ctx_mean * kv_bytes_per_token(cfg)
    achieved = step_bytes / (ms * 1e-3) / 1e9
    e2e_ms, h2d, d2h = time_e2e(model, cfg, args.batch, args.steps, warmup)

    T, d = PREFILL_TOKENS, cfg.head_dim
    flops = 2 * T * layer_params + 2 * head_params \
        + cfg.num_hidden_layers * 2 * cfg.num_attention_heads * d * T * (T + 1)  # QK^T and PV, causal
    pre_frac = flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12)

    points = {}
    if not args.no_points:
        for b in (1, 64):
            pms, _, _, _, check = time_decode(model, cfg, b, max(10, args.steps // 2), warmup)
            points[f"decode_b{b}"] = round(b / (pms * 1e-3), 1)
            graph_check[f"b{b}"] = check

    workloads = {}
    if not args.no_workloads:
        del model
        torch.cuda.empty_cache()
        for name, fn in (("llama_1b_continuous_batching", workload_1b_continuous_batching),
                         ("llama_8b_long_context", workload_8b_long_context)):
            try:
                workloads[name] = fn(pk)
            except Exception as e:   # the headline stands without them; say what went wrong
                workloads[name] = {"error": f"{type(e).__name__}: {e}"[:300]}
                torch.cuda.empty_cache()

    line = {
        "metric": "decode tok/s, Llama 3.2 3B shape, batch 8, context 2048 (1 GPU)",
        "value": round(args.batch / (ms * 1e-3), 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": warmup, "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02) seed 0, uniform-random token ids",
        "impl": "ours",
        "config": {
            "model": "llama-3.2-3b-shape", "layers": cfg.num_hidden_layers,
            "layers_of_full_model": full_layers, "hidden": cfg.hidden_size,
            "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size,
            "vocab": cfg.vocab_size, "global_batch": args.batch, "seq_len": DECODE_CONTEXT,
            "max_context": MAX_CONTEXT, "page_size": PAGE_SIZE, "prefill_tokens": PREFILL_TOKENS,
            "parallelism": "single-gpu", "cuda_graph": True,
            "l2": "inputs larger than L2: every step streams the weights (GBs) once",
            "peaks": pk_src,
        },
        "e2e": {"value": round(args.batch / (e2e_ms * 1e-3), 1), "unit": "tokens/s",
                "ms_per_step": round(e2e_ms, 4), "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "prefill": {"value": round(T / (pre_ms * 1e-3), 1), "tokens": T, "ms": round(pre_ms, 3),
                    "frac": round(pre_frac, 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "workloads": workloads,
        "graph_check": graph_check,
        "clocks": clocks,
    }
    print(json.dumps(line))
    if not all(c["ok"] for c in graph_check.values()):
        print("bench.py: a decode graph's logits part from the eager step's", file=sys.stderr)
        return 3
    return 0


if __name__ == "__main__":
    sys.exit(main())
