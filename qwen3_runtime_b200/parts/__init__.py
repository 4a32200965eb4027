from . import attention, block, feed_forward, norm, position  # noqa: F401  (register the built-in parts)
from .base import (
    BuildContext,
    ParamSpec,
    Part,
    ResidualStream,
    StepContext,
    build_part,
    register_part,
    unregister_part,
)
from .model import DecoderModel

__all__ = [
    "BuildContext",
    "DecoderModel",
    "ParamSpec",
    "Part",
    "ResidualStream",
    "StepContext",
    "build_part",
    "register_part",
    "unregister_part",
]
