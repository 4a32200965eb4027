from .engine_config import EngineConfig, canonical_dtype
from .model_config import ConfigError, Qwen3Config
from .registry import (
    Architecture,
    architecture_for_config,
    default_architecture,
    load_config,
    read_config_json,
    register_architecture,
    registered_architectures,
    resolve_architecture,
    unregister_architecture,
)
from .spec import LayerRun, ModelSpec, PartSpec

__all__ = [
    "Architecture",
    "architecture_for_config",
    "default_architecture",
    "ConfigError",
    "EngineConfig",
    "LayerRun",
    "ModelSpec",
    "PartSpec",
    "Qwen3Config",
    "canonical_dtype",
    "load_config",
    "read_config_json",
    "register_architecture",
    "registered_architectures",
    "resolve_architecture",
    "unregister_architecture",
]
