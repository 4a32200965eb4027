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
    # a small configuration of this architecture for the model-less mode of the Python entry
    # point (random weights, no files); None: the architecture offers none
    tiny_config: Callable[[], Any] | None = None


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class: type, build_spec: Callable[[Any], ModelSpec], *,
                          tiny_config: Callable[[], Any] | None = None) -> None:
    if name in _ARCHITECTURES:
        raise ValueError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = Architecture(name, config_class, build_spec, tiny_config)


def architecture_for_config(config: Any) -> Architecture:
    """The registry entry whose typed config class ``config`` is an instance of (the first
    registered one, if several architectures share a config class)."""
    _ensure_builtin()
    for arch in _ARCHITECTURES.values():
        if type(config) is arch.config_class:
            return arch
    raise ConfigError(f"no registered architecture has the config class {type(config).__name__}")


def default_architecture() -> Architecture:
    """The architecture a model-less run uses when none is named: the first registered one
    that offers a tiny configuration."""
    _ensure_builtin()
    for arch in _ARCHITECTURES.values():
        if arch.tiny_config is not None:
            return arch
    raise ConfigError("no registered architecture offers a tiny configuration")


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


def check_against_pin(config: Any, pinned: Any, pin_path: str | Path) -> None:
    """The model a deployment expects, as a pinned config.json: every size that decides the
    tensors' shapes and the arithmetic has to agree (qwen3_runtime/utils/loader.py:20-30, 57-60
    compares the raw keys; here the typed configs, so a defaulted ``head_dim`` counts too).
    ``max_position_embeddings`` and the norms' eps may differ, as in the reference."""
    keys = getattr(config, "pin_fields", None) or [f for f in vars(config)]
    wrong = [f"{k}={getattr(config, k)!r} (pin {getattr(pinned, k)!r})" for k in keys
             if getattr(config, k) != getattr(pinned, k)]
    if wrong:
        raise ConfigError(f"config.json does not match the pinned model {pin_path}: " + ", ".join(wrong))


def load_config(model_dir: str | Path, pin_path: str | Path | None = None) -> tuple[Architecture, Any]:
    """``(architecture, typed config)`` for a model folder; with ``pin_path`` (a config.json of
    the model that is expected) a folder that holds another model is refused."""
    raw = read_config_json(model_dir)
    arch = resolve_architecture(raw)
    config = arch.config_class.from_hf_config(raw)
    if pin_path is not None:
        pin_raw = json.loads(Path(pin_path).read_text())
        check_against_pin(config, resolve_architecture(pin_raw).config_class.from_hf_config(pin_raw), pin_path)
    return arch, config
