"""Random-weights mode: makes a model folder from a configuration and a seed.

``write_random_model`` writes ``config.json`` and ``model.safetensors`` with
matrices drawn from N(0, std) and norm gains from 1 + N(0, gain_std).  Each
tensor has a generator of its own, seeded from the seed and the tensor's name,
so a tensor's values do not depend on which other tensors exist or in what
order they are made.  (The reference has no such mode; its tests fill every
parameter with N(0, 0.02) under one global seed,
``serving/test_paged_kv_cache.py:204-208``.)

``random_tensors`` makes the same kind of tensors directly on a device, for a
model too large to be worth writing to disk (the benchmark).
"""

from __future__ import annotations

import json
import zlib
from pathlib import Path
from typing import Any

import torch
from safetensors.torch import save_file

from ..config.registry import architecture_of
from ..parts.base import Runtime, TensorSpec
from .loader import target_dtype

_STORE_DTYPES = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}


def _tensor_seed(seed: int, name: str) -> int:
    return (int(seed) * 0x9E3779B1 + zlib.crc32(name.encode())) & 0x7FFFFFFFFFFFFFFF


def _draw(name: str, spec: TensorSpec, seed: int, std: float, gain_std: float,
          device: torch.device) -> torch.Tensor:
    if spec.kind == "table":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    gen = torch.Generator(device=device)
    gen.manual_seed(_tensor_seed(seed, name))
    if spec.init == "zeros":
        return torch.zeros(spec.shape, dtype=torch.float32, device=device)
    t = torch.randn(spec.shape, generator=gen, dtype=torch.float32, device=device)
    if spec.init == "gain":
        return 1.0 + gain_std * t
    return std * t


def model_for_config(config: dict[str, Any]):
    """(typed config, DecoderModel without weights) for a config.json dictionary."""
    from ..models.plan import DecoderModel
    arch = architecture_of(config)
    cfg = arch.config_class.from_dict(config)
    return cfg, DecoderModel(arch.plan(cfg))


def write_random_model(folder: str | Path, config: dict[str, Any], seed: int,
                       std: float = 0.02, gain_std: float = 0.1) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` under ``folder``."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    cfg, model = model_for_config(config)
    store = _STORE_DTYPES[getattr(cfg, "torch_dtype", "bfloat16")]
    tensors = {}
    for name, spec in model.tensor_specs().items():
        t = _draw(name, spec, seed, std, gain_std, torch.device("cpu"))
        tensors[name] = t if spec.kind == "table" else t.to(store)
    save_file(tensors, str(folder / "model.safetensors"))
    with open(folder / "config.json", "w") as f:
        json.dump(cfg.to_dict(), f, indent=1)
    return folder


def random_tensors(specs: dict[str, TensorSpec], seed: int, rt: Runtime, store: torch.dtype,
                   std: float = 0.02, gain_std: float = 0.1) -> dict[str, torch.Tensor]:
    """The tensors of ``specs`` drawn on ``rt.device``, rounded to ``store`` first."""
    out = {}
    for name, spec in specs.items():
        t = _draw(name, spec, seed, std, gain_std, rt.device)
        if spec.kind != "table":
            t = t.to(store).to(target_dtype(spec, store, rt))
        out[name] = t.contiguous()
    return out
