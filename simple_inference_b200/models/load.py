"""From a model folder (or a configuration and a seed) to a model with weights bound."""

from __future__ import annotations

from pathlib import Path
from typing import Any

import torch

from ..config.model_config import ModelConfig
from ..config.registry import architecture_of, read_config
from ..parts.base import Runtime
from ..weights.loader import load_tensors
from ..weights.random_init import _STORE_DTYPES, random_tensors
from .plan import DecoderModel

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
           "float32": torch.float32, "fp32": torch.float32}


def runtime_for(dtype: str | torch.dtype, device: str | torch.device = "cuda") -> Runtime:
    if isinstance(dtype, str):
        if dtype not in _DTYPES:
            raise ValueError(f"dtype {dtype!r}: choose bfloat16 or float32")
        dtype = _DTYPES[dtype]
    if dtype not in (torch.bfloat16, torch.float32):
        raise ValueError(f"dtype {dtype}: choose bfloat16 or float32")
    return Runtime(torch.device(device), dtype)


def load_model(model_dir: str | Path, dtype: str | torch.dtype = "bfloat16",
               device: str | torch.device = "cuda") -> tuple[ModelConfig, DecoderModel]:
    """Read ``config.json``, pick the architecture from it, load and bind the weights."""
    rt = runtime_for(dtype, device)
    arch, cfg = read_config(model_dir)
    model = DecoderModel(arch.plan(cfg))
    tensors = load_tensors(model_dir, model.tensor_specs(), model.optional_tensor_names(), rt)
    model.bind(tensors, rt)
    return cfg, model


def random_model(config: dict[str, Any], seed: int, dtype: str | torch.dtype = "bfloat16",
                 device: str | torch.device = "cuda") -> tuple[ModelConfig, DecoderModel]:
    """A model with random weights drawn on the device (nothing is written to disk)."""
    rt = runtime_for(dtype, device)
    arch = architecture_of(config)
    cfg = arch.config_class.from_dict(config)
    model = DecoderModel(arch.plan(cfg))
    store = _STORE_DTYPES[getattr(cfg, "torch_dtype", "bfloat16")]
    model.bind(random_tensors(model.tensor_specs(), seed, rt, store), rt)
    return cfg, model
