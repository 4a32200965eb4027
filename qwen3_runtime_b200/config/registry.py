"""One registry from an architecture's name (``config.json: architectures``) to its model.

An entry gives the typed config class and the function that turns a config into
a :class:`ModelSpec`.  Adding an architecture is one ``register_architecture``
call; the reference hard-wires its single class instead
(qwen3_runtime/models/qwen3.py:35-37).
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Mapping

from .model_config import ConfigError
from .spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type
    build_spec: Callable[[Any], ModelSpec]


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class: type, build_spec: Callable[[Any], ModelSpec]) -> None:
    if name in _ARCHITECTURES:
        raise ValueError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = Architecture(name, config_class, build_spec)


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def registered_architectures() -> list[str]:
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def _ensure_builtin() -> None:
    from .. import models  # noqa: F401  (registers the built-in architecture)


def resolve_architecture(raw: Mapping[str, Any]) -> Architecture:
    """Pick the registered architecture named in ``raw['architectures']``."""
    _ensure_builtin()
    names = raw.get("architectures") or []
    for name in names:
        if name in _ARCHITECTURES:
            return _ARCHITECTURES[name]
    raise ConfigError(f"unsupported architectures: {list(names)} (registered: {sorted(_ARCHITECTURES)})")


def read_config_json(model_dir: str | Path) -> dict[str, Any]:
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"no config.json in {model_dir}")
    return json.loads(path.read_text())


def load_config(model_dir: str | Path) -> tuple[Architecture, Any]:
    """``(architecture, typed config)`` for a model folder."""
    raw = read_config_json(model_dir)
    arch = resolve_architecture(raw)
    return arch, arch.config_class.from_hf_config(raw)
