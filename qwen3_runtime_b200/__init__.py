"""A single-GPU inference engine for Qwen3 dense, written for NVIDIA B200 (sm_100a).

Public entry points: :class:`LLM` (``generate``), :func:`build_engine`,
:class:`SamplingParams`, and ``python -m qwen3_runtime_b200.cli``.
"""

from .config import EngineConfig, Qwen3Config
from .sampling.params import SamplingParams

__all__ = ["EngineConfig", "LLM", "Qwen3Config", "SamplingParams", "build_engine"]


def __getattr__(name: str):
    if name == "LLM":
        from .llm import LLM

        return LLM
    if name == "build_engine":
        from .engine.factory import build_engine

        return build_engine
    raise AttributeError(name)
