#!/usr/bin/env python3
"""Command line of the engine: one prompt of token ids in, generated token ids out.

The counterpart of the reference's ``generate.py`` (``generate.py:245-315``),
which runs a hard-coded prompt with ``max_seq_len=4096``, ``max_new_tokens=2048``
and ``{temperature 0.7, top_k 50, top_p 0.9}``, prints a metrics table and writes
``metrics/run_NNN.json`` (``utilities.py:41-70``).  Here everything is an option;
the options keep the reference's names (``max_new_tokens``, ``temperature``,
``top_k``, ``top_p`` of ``generate()``, ``generate.py:50-59``; ``max_running``,
``max_seq_len``, ``block_size``, ``num_kv_blocks``, ``token_budget``, ``eos_id``
of ``InferenceEngine``, ``serving/engine.py:96-113``) and the defaults of the
reference's ``generate()``: temperature 1.0, top_k 50, top_p 0.9, 256 new tokens.
Prompts are token ids: the reference's tokenizer wraps files that have to be
downloaded (``tokenizer.py:46-72``), which this engine does not do.

    python generate.py --model DIR --prompt-ids 1,15,27 --max-new-tokens 32
    python generate.py --random-config cfg.json --seed 0 --prompt-len 64 --temperature 0
"""

from __future__ import annotations

import argparse
import datetime
import json
import sys
import tempfile
from pathlib import Path


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    src = ap.add_mutually_exclusive_group(required=True)
    src.add_argument("--model", help="folder with config.json and model.safetensors")
    src.add_argument("--random-config", help="config.json of a model to fill with random weights")
    ap.add_argument("--seed", type=int, default=0, help="seed of random weights and of sampling")
    ap.add_argument("--save-random-model", help="with --random-config: keep the model folder here")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    pr = ap.add_mutually_exclusive_group()
    pr.add_argument("--prompt-ids", help="comma-separated token ids")
    pr.add_argument("--prompt-file", help="file with token ids separated by spaces or commas")
    pr.add_argument("--prompt-len", type=int, help="a random prompt of this many ids (seeded)")
    ap.add_argument("--max-new-tokens", type=int, default=256)
    ap.add_argument("--temperature", type=float, default=1.0, help="0 = greedy")
    ap.add_argument("--top-k", type=int, default=50, help="0 = off")
    ap.add_argument("--top-p", type=float, default=0.9, help="1.0 = off")
    ap.add_argument("--eos-id", type=int, default=None, help="stop token; -1 = never stop")
    ap.add_argument("--max-running", type=int, default=1)
    ap.add_argument("--max-seq-len", type=int, default=4096)
    ap.add_argument("--block-size", type=int, default=16, help="tokens per cache page")
    ap.add_argument("--num-kv-blocks", type=int, default=None)
    ap.add_argument("--token-budget", type=int, default=None)
    ap.add_argument("--chunk-size", type=int, default=None, help="longest prompt portion per step")
    ap.add_argument("--max-tokens-per-step", type=int, default=None)
    ap.add_argument("--no-cuda-graphs", action="store_true")
    ap.add_argument("--stats-json", help="write the timing record here "
                                         "(default: metrics/run_NNN.json when --metrics-dir is given)")
    ap.add_argument("--metrics-dir", help="folder for numbered run_NNN.json records")
    ap.add_argument("--quiet", action="store_true", help="do not stream tokens to stderr")
    return ap.parse_args(argv)


def next_run_path(metrics_dir: Path) -> Path:
    """metrics_dir/run_000.json, run_001.json, ...: one past the highest present."""
    metrics_dir.mkdir(parents=True, exist_ok=True)
    taken = [int(p.stem.split("_")[1]) for p in metrics_dir.glob("run_*.json")
             if p.stem.split("_")[1].isdigit()]
    return metrics_dir / f"run_{(max(taken) + 1 if taken else 0):03d}.json"


def print_metrics_table(stats: dict) -> None:
    rows = [("TTFT ms (time to 1st tok)", "ttft_ms"), ("TPOT ms (per output tok)", "tpot_ms"),
            ("decode tok/s (1000/TPOT)", "decode_tok_s"), ("prefill ms", "prefill_ms"),
            ("prompt tokens", "prompt_tokens"), ("new tokens", "new_tokens"),
            ("total tok/s", "total_tok_s"), ("total wall ms", "total_wall_ms"),
            ("peak VRAM GB", "peak_vram_gb")]
    print("=" * 60, file=sys.stderr)
    for label, key in rows:
        print(f"  {label:<26}: {stats.get(key, 0):>12}", file=sys.stderr)
    print("=" * 60, file=sys.stderr)


def main(argv=None) -> int:
    args = parse_args(argv)
    import torch
    from simple_inference_b200 import InferenceEngine, read_config, write_random_model

    if not torch.cuda.is_available():
        print("generate.py: no CUDA device; the engine has no CPU path", file=sys.stderr)
        return 2
    keep = None
    if args.random_config:
        with open(args.random_config) as f:
            config = json.load(f)
        if args.save_random_model:
            model_dir = write_random_model(args.save_random_model, config, args.seed)
        else:
            keep = tempfile.TemporaryDirectory(prefix="si_b200_model_")
            model_dir = write_random_model(keep.name, config, args.seed)
    else:
        model_dir = Path(args.model)
    _, cfg = read_config(model_dir)

    if args.prompt_ids:
        prompt = [int(x) for x in args.prompt_ids.replace(",", " ").split()]
    elif args.prompt_file:
        prompt = [int(x) for x in Path(args.prompt_file).read_text().replace(",", " ").split()]
    else:
        g = torch.Generator().manual_seed(args.seed)
        prompt = torch.randint(0, cfg.vocab_size, (args.prompt_len or 16,), generator=g).tolist()

    engine = InferenceEngine.from_folder(
        model_dir, args.dtype, "cuda", max_running=args.max_running,
        max_seq_len=min(args.max_seq_len, cfg.max_position_embeddings),
        block_size=args.block_size, num_kv_blocks=args.num_kv_blocks,
        token_budget=args.token_budget, eos_id=args.eos_id, temperature=args.temperature,
        top_k=args.top_k, top_p=args.top_p, use_cuda_graphs=not args.no_cuda_graphs,
        max_tokens_per_step=args.max_tokens_per_step, chunk_size=args.chunk_size, seed=args.seed)

    def on_token(tok: int) -> None:
        if not args.quiet:
            print(tok, end=" ", file=sys.stderr, flush=True)

    tokens, stats = engine.generate_with_stats(prompt, args.max_new_tokens, on_token=on_token)
    if not args.quiet:
        print(file=sys.stderr)
        print_metrics_table(stats)
    record = {
        "timestamp": datetime.datetime.now(datetime.timezone.utc).isoformat(timespec="seconds"),
        "model_id": str(model_dir), "backend": f"sm_100a kernels, {args.dtype}",
        "device": torch.cuda.get_device_name(0),
        "sampling": {"temperature": args.temperature, "top_k": args.top_k, "top_p": args.top_p,
                     "seed": args.seed},
        "metrics": stats,
    }
    path = Path(args.stats_json) if args.stats_json else (
        next_run_path(Path(args.metrics_dir)) if args.metrics_dir else None)
    if path is not None:
        path.parent.mkdir(parents=True, exist_ok=True)
        path.write_text(json.dumps(record, indent=2))
    print(json.dumps({"tokens": tokens, "finish": "length" if len(tokens) == args.max_new_tokens else "stop"}))
    if keep is not None:
        keep.cleanup()
    return 0


if __name__ == "__main__":
    sys.exit(main())
