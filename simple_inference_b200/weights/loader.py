"""Weights from safetensors, bound by tensor name.

A model folder holds ``config.json`` and either ``model.safetensors`` or
shards named by ``model.safetensors.index.json`` (the two layouts the
reference reads, ``loader.py:179-203``).  The model says which tensors it needs
and with what shape (``DecoderModel.tensor_specs``); the loader compares that
with what the files hold and raises ONE ``WeightError`` that lists every
missing tensor, every unexpected tensor and every wrong shape or dtype.  (The
reference raises on the first missing name only, ``loader.py:220-224``, checks
no shapes and swallows every error around ``lm_head``, ``model/llama.py:147-154``.)

dtypes: operands of matrix products are held in the compute dtype (bfloat16
when serving, float32 on the 32-bit path).  Small tensors (gains) keep bfloat16
or 32-bit as stored when serving and are float32 on the 32-bit path.  Integer
tables are int32.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch
from safetensors import safe_open

from ..parts.base import Runtime, TensorSpec

_FLOAT_DTYPES = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16}
_INT_DTYPES = {"I32": torch.int32, "I64": torch.int64}


class WeightError(RuntimeError):
    """The checkpoint does not fit the model.  Lists everything that is wrong."""

    def __init__(self, model_dir, missing, unexpected, wrong):
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong = sorted(wrong)
        lines = [f"weights in {model_dir} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong:
            lines.append(f"  wrong shape or dtype ({len(self.wrong)}):")
            lines.extend(f"    {w}" for w in self.wrong)
        super().__init__("\n".join(lines))


def _shard_map(model_dir: Path) -> dict[str, Path]:
    """tensor name -> file that holds it."""
    index = model_dir / "model.safetensors.index.json"
    if index.is_file():
        with open(index) as f:
            weight_map = json.load(f)["weight_map"]
        return {name: model_dir / shard for name, shard in weight_map.items()}
    single = model_dir / "model.safetensors"
    if not single.is_file():
        raise FileNotFoundError(f"{model_dir} holds neither model.safetensors nor "
                                f"model.safetensors.index.json")
    with safe_open(str(single), framework="pt", device="cpu") as f:
        return {name: single for name in f.keys()}


def target_dtype(spec: TensorSpec, stored: torch.dtype, rt: Runtime) -> torch.dtype:
    if spec.kind == "table":
        return torch.int32
    if rt.is_fp32:
        return torch.float32
    if spec.kind == "matrix":
        return rt.dtype
    return torch.float32 if stored == torch.float32 else torch.bfloat16


def load_tensors(model_dir: str | Path, specs: dict[str, TensorSpec], optional: set[str],
                 rt: Runtime) -> dict[str, torch.Tensor]:
    """Read every tensor of ``specs`` onto ``rt.device`` in its final dtype."""
    model_dir = Path(model_dir)
    where = _shard_map(model_dir)
    missing = [n for n in specs if n not in where]
    unexpected = [n for n in where if n not in specs and n not in optional]
    wrong: list[str] = []

    handles: dict[Path, object] = {}

    def handle(path: Path):
        if path not in handles:
            if not path.is_file():
                raise FileNotFoundError(f"shard {path} named by the index does not exist")
            handles[path] = safe_open(str(path), framework="pt", device="cpu")
        return handles[path]

    for name, spec in specs.items():
        if name not in where:
            continue
        sl = handle(where[name]).get_slice(name)
        shape, dt = tuple(sl.get_shape()), sl.get_dtype()
        if shape != tuple(spec.shape):
            wrong.append(f"{name}: shape {shape}, the model needs {tuple(spec.shape)}")
        allowed = _INT_DTYPES if spec.kind == "table" else _FLOAT_DTYPES
        if dt not in allowed:
            wrong.append(f"{name}: dtype {dt}, the model needs one of {sorted(allowed)}")
    if missing or unexpected or wrong:
        raise WeightError(model_dir, missing, unexpected, wrong)

    out: dict[str, torch.Tensor] = {}
    for name, spec in specs.items():
        t = handle(where[name]).get_tensor(name)
        out[name] = t.to(device=rt.device, dtype=target_dtype(spec, t.dtype, rt)).contiguous()
    return out
