"""Runtime knobs of the engine (not of the model).

Parity: qwen3_runtime/config.py:16-24 for the names ``block_size``,
``num_kv_blocks``, ``max_num_seqs``, ``max_num_batched_tokens``,
``eos_token_id`` and ``cuda_graph``; the offload / speculative fields of the
reference have no counterpart here.
"""

from __future__ import annotations

from dataclasses import dataclass

DTYPES = ("bfloat16", "float32")


def canonical_dtype(name: str) -> str:
    """Map the accepted spellings to ``"bfloat16"`` or ``"float32"``."""
    key = str(name).lower().replace("torch.", "")
    table = {"bf16": "bfloat16", "bfloat16": "bfloat16", "fp32": "float32", "float32": "float32", "float": "float32"}
    if key not in table:
        raise ValueError(f"dtype must be one of bfloat16/float32 (bf16/fp32), got {name!r}")
    return table[key]


@dataclass(frozen=True)
class EngineConfig:
    block_size: int = 16  # tokens per KV page
    num_kv_blocks: int | None = None  # pages per cache group; None = size from free memory
    max_num_seqs: int = 8
    max_num_batched_tokens: int = 2048
    eos_token_id: int | None = None
    cuda_graph: bool = True  # replay captured decode steps
    dtype: str = "bfloat16"
    kv_memory_fraction: float = 0.85  # share of free device memory given to the pages
    run_ahead: bool = True  # put the next decode step on the device before reading this one's tokens

    def __post_init__(self) -> None:
        if self.block_size < 1:
            raise ValueError("block_size must be positive")
        if self.num_kv_blocks is not None and self.num_kv_blocks < 1:
            raise ValueError("num_kv_blocks must be positive")
        if self.max_num_seqs < 1:
            raise ValueError("max_num_seqs must be positive")
        if self.max_num_batched_tokens < 1:
            raise ValueError("max_num_batched_tokens must be positive")
        if not 0.0 < self.kv_memory_fraction <= 1.0:
            raise ValueError("kv_memory_fraction must be in (0, 1]")
        object.__setattr__(self, "dtype", canonical_dtype(self.dtype))
