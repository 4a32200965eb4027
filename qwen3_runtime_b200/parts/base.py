"""What every part is, and the registry that finds a part class by category and kind.

Categories: ``norm``, ``position``, ``mixer``, ``feed_forward``, ``block``.  A part is
built from a :class:`PartSpec` (its sizes and constants) and a :class:`BuildContext`
(dtype, device, kernel table); it declares its tensors with :meth:`Part.param_specs`
(names relative to the part's own prefix) and receives them, already on the device,
in :meth:`Part.load`.  Registering a new kind is one :func:`register_part` call, which
a test or an extension can make without touching this package.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

import torch

from ..config.spec import PartSpec

CATEGORIES = ("norm", "position", "mixer", "feed_forward", "block")


@dataclass(frozen=True)
class ParamSpec:
    """A stored tensor a part needs.  ``kind`` decides how it is kept on the device:

    ``matrix``  -- operand of a matrix product or lookup table: the compute dtype;
    ``vector``  -- small per-channel parameter: float32 (a lossless copy of bfloat16
                   storage; a tensor stored in 32-bit stays 32-bit);
    ``int``     -- integer table: int32.
    """

    shape: tuple[int, ...]
    kind: str = "matrix"


@dataclass
class BuildContext:
    dtype: torch.dtype
    device: torch.device
    ops: Any  # the kernel table (qwen3_runtime_b200.ops.cuda.CudaOps in production)
    shared: dict = field(default_factory=dict)  # tables shared between parts (e.g. rotary cos/sin)


@dataclass
class StepContext:
    """The batch of one step as the parts see it (device tensors are int32)."""

    num_tokens: int
    num_seqs: int
    token_ids: torch.Tensor  # [T]
    positions: torch.Tensor  # [T] absolute position of each token in its sequence
    token_seq: torch.Tensor  # [T] row of the batch (sequence) each token belongs to
    cu_seqlens: torch.Tensor  # [B + 1] first token of each sequence in the packed batch
    kv_lens: torch.Tensor  # [B] tokens in the cache after this step
    state_slots: torch.Tensor  # [B] fixed-size state slot of each sequence
    block_tables: list[torch.Tensor]  # per paged cache group: [B, max_pages]
    logit_rows: torch.Tensor  # [R] packed rows whose logits are wanted
    num_logit_rows: int
    max_query_len: int  # host copies of batch extremes, for kernel choice
    max_kv_len: int
    decode_only: bool  # every sequence brings exactly one token
    kv_longest: torch.Tensor | None = None  # [1] the largest of kv_lens, on the device
    single_seqs: torch.Tensor | None = None  # [num_single] sequences that bring exactly one token
    num_single: int = 0
    # host copies (lists) for parts that need them without a device read
    host_cu_seqlens: list[int] = field(default_factory=list)
    host_kv_lens: list[int] = field(default_factory=list)
    # Non-zero in a step that is being captured into (or replayed from) a CUDA graph: the
    # block-table width the graph is made for.  A part whose launch shape depends on the
    # longest sequence has to size it from ``captured_width * page_size`` then, not from
    # ``max_kv_len``, because the graph is replayed for longer sequences of the same width.
    captured_width: int = 0
    # In a step in which every sequence brings one token: what the parts' choosers (Part.step_choosers)
    # answered for the step's lengths, by name.  A captured step is specialised by these values:
    # they are part of its graph's key, and a part must let nothing else about the lengths of the
    # moment decide what it launches.
    choices: dict = field(default_factory=dict)
    extras: dict = field(default_factory=dict)  # per-step scratch shared by the layers of a step


class Part:
    category = ""
    # A norm that can take ``ResidualStream.pending`` as partial sums (see there) says so here.
    adds_partial_sums = False
    # Set on a mixer or feed-forward by whoever arranges the parts, when the norm that will
    # fold its output into the residual sum adds partial sums itself: ``forward`` may then
    # return float32 ``[parts, tokens, hidden]`` whose sum over the first axis is the output.
    partial_sums_ok = False

    def __init__(self, spec: PartSpec, ctx: BuildContext):
        self.spec = spec
        self.ctx = ctx
        self.ops = ctx.ops

    def param_specs(self) -> dict[str, ParamSpec]:
        return {}

    def step_choosers(self) -> dict:
        """``{name: function(kv_lens) -> hashable}``: choices that this part's kernels make from the
        lengths (tokens in the cache after the step, one per sequence) of a step in which every
        sequence brings one token, e.g. into how many slices the keys are cut.  Parts that answer
        with the same name make the same choice; it is worked out once per step and reaches
        ``forward`` as ``step.choices[name]``.  A part made of parts passes its parts' choosers on."""
        return {}

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        if tensors:
            raise ValueError(f"{type(self).__name__} takes no tensors")

    def kernel_groups(self) -> list[str]:
        """CUDA source groups this part launches (compiled before the first step)."""
        return []

    def position_limit(self) -> int | None:
        """Positions this part can serve (``0 .. limit - 1``), or None when any position will do.
        A position encoding with a table says its length; a part made of parts passes on the
        smallest limit among them."""
        return None


_REGISTRY: dict[tuple[str, str], Callable[[PartSpec, BuildContext], Part]] = {}


def register_part(category: str, kind: str, factory: Callable[[PartSpec, BuildContext], Part],
                  *, replace: bool = False) -> None:
    if category not in CATEGORIES:
        raise ValueError(f"unknown part category {category!r}; one of {CATEGORIES}")
    if (category, kind) in _REGISTRY and not replace:
        raise ValueError(f"{category} part {kind!r} is already registered")
    _REGISTRY[(category, kind)] = factory


def unregister_part(category: str, kind: str) -> None:
    _REGISTRY.pop((category, kind), None)


def build_part(category: str, spec: PartSpec, ctx: BuildContext) -> Part:
    try:
        factory = _REGISTRY[(category, spec.kind)]
    except KeyError:
        known = sorted(k for c, k in _REGISTRY if c == category)
        raise ValueError(f"no {category} part of kind {spec.kind!r} is registered (known: {known})") from None
    return factory(spec, ctx)


class ResidualStream:
    """The residual sum of a step, kept in float32, plus what has not been added yet.

    ``pending`` is the output of the last sublayer; the next norm adds it to ``resid``
    and normalises in one kernel.  It is ``[tokens, hidden]`` in the compute dtype, or float32
    ``[parts, tokens, hidden]``: partial sums of the sublayer's last product over ranges of
    its inner dimension, which the norm adds in order (one kernel less waits for the sum).  A fresh stream holds an embedding lookup instead of
    values: the first norm gathers the rows, stores them as ``resid`` and normalises.
    """

    def __init__(self, num_tokens: int, hidden_size: int, *, ids: torch.Tensor, table: torch.Tensor):
        self.num_tokens = num_tokens
        self.hidden_size = hidden_size
        self.embed: tuple[torch.Tensor, torch.Tensor] | None = (ids, table)
        self.resid: torch.Tensor | None = None
        self.pending: torch.Tensor | None = None
