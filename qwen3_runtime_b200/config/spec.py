"""Architecture-neutral description of a model as data.

A model is a list of blocks, each made of parts (mixer, feed-forward, norms,
position encoding), and a *run order*: which block runs when and which cache it
reads and writes.  Parts are named by ``kind`` and carry their own sizes and
constants, so one model may use different mixers or feed-forwards in different
layers, and no part knows which model it is in.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass(frozen=True)
class PartSpec:
    """One part: its registered ``kind`` and the parameters that part understands."""

    kind: str
    params: dict[str, Any] = field(default_factory=dict)

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerRun:
    """One entry of the run order.

    ``block`` indexes ``ModelSpec.blocks`` (a block may be named twice: its
    weights are shared).  ``cache`` is the id of the cache layer the mixer uses;
    two entries with the same ``cache`` share keys and values.  ``writes`` says
    whether this entry stores its own keys/values (or state) there or only reads
    what an earlier entry stored.
    """

    block: int
    cache: int
    writes: bool = True


@dataclass(frozen=True)
class ModelSpec:
    vocab_size: int
    hidden_size: int
    blocks: tuple[PartSpec, ...]
    order: tuple[LayerRun, ...]
    final_norm: PartSpec
    tie_word_embeddings: bool
    embed_name: str = "model.embed_tokens.weight"
    head_name: str = "lm_head.weight"
    block_prefix: str = "model.layers.{index}."
    final_norm_prefix: str = "model.norm."
    # the head's epilogue: logits * logit_scale, then (if set) softcap * tanh(logits / softcap)
    logit_scale: float = 1.0
    logit_softcap: float | None = None

    def __post_init__(self) -> None:
        if self.logit_softcap is not None and not self.logit_softcap > 0:
            raise ValueError("logit_softcap must be positive (or None)")
        writers: set[int] = set()
        for run in self.order:
            if not 0 <= run.block < len(self.blocks):
                raise ValueError(f"run order names block {run.block}; the model has {len(self.blocks)}")
            if run.writes:
                if run.cache in writers:
                    raise ValueError(f"cache layer {run.cache} is written by two run entries")
                writers.add(run.cache)
            elif run.cache not in writers:
                raise ValueError(f"run entry reads cache layer {run.cache} before any entry writes it")

    @staticmethod
    def sequential_order(num_blocks: int) -> tuple[LayerRun, ...]:
        return tuple(LayerRun(block=i, cache=i) for i in range(num_blocks))
