"""One registry from an architecture's name to its configuration class and model plan.

The name is ``config.json["architectures"][0]``.  The reference has no
registry: every entry point imports ``LlamaModel`` by name and ignores
config.json (``model/llama.py:335``, ``generate.py:273``).
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable

from .model_config import ConfigError, ModelConfig


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type[ModelConfig]
    plan: Callable[[Any], Any]  # typed config -> models.plan.ModelPlan


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class: type[ModelConfig],
                          plan: Callable[[Any], Any]) -> None:
    _ARCHITECTURES[name] = Architecture(name, config_class, plan)


def known_architectures() -> list[str]:
    _load_builtin()
    return sorted(_ARCHITECTURES)


def _load_builtin() -> None:
    from .. import models  # noqa: F401  (importing registers the built-in architectures)


def architecture_of(config: dict[str, Any]) -> Architecture:
    _load_builtin()
    names = config.get("architectures")
    if not names or not isinstance(names, (list, tuple)):
        raise ConfigError("config.json has no 'architectures' list; "
                          f"known architectures: {sorted(_ARCHITECTURES)}")
    name = names[0]
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(f"architecture {name!r} is not registered; "
                          f"known architectures: {sorted(_ARCHITECTURES)}") from None


def read_config(model_dir: str | Path) -> tuple[Architecture, ModelConfig]:
    """Read ``model_dir/config.json`` into the typed configuration of its architecture."""
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"{path} does not exist")
    with open(path) as f:
        raw = json.load(f)
    arch = architecture_of(raw)
    return arch, arch.config_class.from_dict(raw)
