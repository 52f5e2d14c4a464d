"""Typed model configuration read from a checkpoint's ``config.json``.

Every size and constant of the model comes from here; no other module holds a
model dimension.  The key set follows the reference's ``ModelConfig``
(``config.py:39-109``) and ``RopeScalingConfig`` (``config.py:19-36``), with
three differences that the reference's own code needs but does not honour:
``head_dim`` may be given explicitly, ``rope_scaling`` may be null (the
reference crashes on it, ``model/llama.py:77-86``) and ``tie_word_embeddings``
is consulted (the reference parses and ignores it, ``config.py:107``).
"""

from __future__ import annotations

import json
from dataclasses import MISSING as _MISSING
from dataclasses import dataclass, fields
from pathlib import Path
from typing import Any, ClassVar


class ConfigError(ValueError):
    """A config.json that cannot describe a model this framework can run."""


@dataclass(frozen=True)
class RopeScaling:
    """``rope_scaling`` of config.json (reference ``config.py:19-36``).

    Only ``rope_type == "llama3"`` changes the frequencies; every other type is
    plain rotary encoding, as in the reference (``ops/rope.py:101``).
    """

    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "RopeScaling":
        rope_type = d.get("rope_type", d.get("type", "default"))
        if rope_type == "llama3":
            missing = [k for k in ("factor", "low_freq_factor", "high_freq_factor",
                                   "original_max_position_embeddings") if k not in d]
            if missing:
                raise ConfigError(f"rope_scaling of type llama3 lacks keys {missing}")
        return cls(
            rope_type=str(rope_type),
            factor=float(d.get("factor", 1.0)),
            low_freq_factor=float(d.get("low_freq_factor", 1.0)),
            high_freq_factor=float(d.get("high_freq_factor", 4.0)),
            original_max_position_embeddings=int(d.get("original_max_position_embeddings", 0)),
        )

    def to_dict(self) -> dict[str, Any]:
        return {
            "rope_type": self.rope_type,
            "factor": self.factor,
            "low_freq_factor": self.low_freq_factor,
            "high_freq_factor": self.high_freq_factor,
            "original_max_position_embeddings": self.original_max_position_embeddings,
        }


# dtypes a checkpoint may be stored in (reference ``config.py:137-142``); a float16
# checkpoint is converted when it is loaded and served in bfloat16
_DTYPE_NAMES = ("bfloat16", "float16", "float32")


@dataclass(kw_only=True)
class ModelConfig:
    """Base of every architecture's typed configuration.

    A subclass lists its config.json keys as dataclass fields.  Fields without
    a default are required; ``from_dict`` reports all missing ones at once.
    """

    architectures: tuple[str, ...] = ()

    # keys whose value is a nested object with its own class
    _nested: ClassVar[dict[str, Any]] = {}

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "ModelConfig":
        known = {f.name: f for f in fields(cls) if f.init}
        missing = [
            name for name, f in known.items()
            if name not in d and f.default is _MISSING and f.default_factory is _MISSING
        ]
        if missing:
            raise ConfigError(
                f"config.json lacks required keys for {cls.__name__}: {sorted(missing)}"
            )
        kwargs: dict[str, Any] = {}
        for name in known:
            if name not in d:
                continue
            value = d[name]
            nested = cls._nested.get(name)
            if nested is not None and value is not None:
                value = nested.from_dict(value)
            if name == "architectures":
                value = tuple(value)
            kwargs[name] = value
        cfg = cls(**kwargs)
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path: str | Path) -> "ModelConfig":
        with open(path) as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {}
        for f in fields(self):
            if not f.init:
                continue
            v = getattr(self, f.name)
            if hasattr(v, "to_dict"):
                v = v.to_dict()
            elif isinstance(v, tuple):
                v = list(v)
            out[f.name] = v
        return out

    def validate(self) -> None:  # pragma: no cover - overridden
        pass



@dataclass(kw_only=True)
class LlamaConfig(ModelConfig):
    """config.json of ``LlamaForCausalLM`` (reference ``config.py:84-109``).

    Required keys are the reference's ten required keys.  ``head_dim`` defaults
    to ``hidden_size // num_attention_heads`` (``config.py:81``);
    ``tie_word_embeddings`` defaults to True and ``torch_dtype`` to bfloat16 as
    in ``config.py:107-108``.  Token ids have no default: a checkpoint without
    ``eos_token_id`` never stops on a token.
    """

    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    vocab_size: int
    num_attention_heads: int
    num_key_value_heads: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    rope_scaling: RopeScaling | None = None
    head_dim: int | None = None
    bos_token_id: int | None = None
    eos_token_id: int | list[int] | None = None
    tie_word_embeddings: bool = True
    torch_dtype: str = "bfloat16"
    hidden_act: str = "silu"
    attention_bias: bool = False
    mlp_bias: bool = False

    _nested: ClassVar[dict[str, Any]] = {"rope_scaling": RopeScaling}

    def validate(self) -> None:
        ints = ("hidden_size", "intermediate_size", "num_hidden_layers", "vocab_size",
                "num_attention_heads", "num_key_value_heads", "max_position_embeddings")
        for name in ints:
            v = getattr(self, name)
            if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
                raise ConfigError(f"{name} must be a positive integer, got {v!r}")
        if self.head_dim is None:
            # reference config.py:73-81
            if self.hidden_size % self.num_attention_heads != 0:
                raise ConfigError(
                    f"hidden_size {self.hidden_size} is not divisible by "
                    f"num_attention_heads {self.num_attention_heads} and no head_dim is given"
                )
            self.head_dim = self.hidden_size // self.num_attention_heads
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                f"num_attention_heads {self.num_attention_heads} is not divisible by "
                f"num_key_value_heads {self.num_key_value_heads}"
            )
        if self.head_dim <= 0 or self.head_dim % 2 != 0:
            raise ConfigError(f"head_dim must be positive and even, got {self.head_dim}")
        if not (float(self.rms_norm_eps) > 0.0):
            raise ConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps!r}")
        if not (float(self.rope_theta) > 0.0):
            raise ConfigError(f"rope_theta must be positive, got {self.rope_theta!r}")
        self.rope_theta = float(self.rope_theta)
        self.rms_norm_eps = float(self.rms_norm_eps)
        if self.torch_dtype not in _DTYPE_NAMES:
            raise ConfigError(
                f"torch_dtype {self.torch_dtype!r} is not one of {_DTYPE_NAMES}"
            )
        if self.hidden_act != "silu":
            raise ConfigError(f"hidden_act {self.hidden_act!r}: only 'silu' is built")
        if self.attention_bias or self.mlp_bias:
            raise ConfigError("attention_bias / mlp_bias are not built (the reference has none)")
        rs = self.rope_scaling
        if rs is not None and rs.rope_type == "llama3":
            if rs.factor <= 0 or rs.original_max_position_embeddings <= 0:
                raise ConfigError("llama3 rope_scaling needs positive factor and original length")
            if rs.high_freq_factor == rs.low_freq_factor:
                raise ConfigError("llama3 rope_scaling needs high_freq_factor != low_freq_factor")

    @property
    def num_kv_groups(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    def eos_ids(self) -> tuple[int, ...]:
        if self.eos_token_id is None:
            return ()
        if isinstance(self.eos_token_id, int):
            return (self.eos_token_id,)
        return tuple(int(x) for x in self.eos_token_id)
