"""A request as the engine tracks it.

What a request *is* -- its tokens so far, its sampling parameters and its stop
conditions -- lives here; what it *holds* (pages in every cache group, a state slot,
how many of its tokens are in the cache) lives in the :class:`RequestCache` handle that
the cache manager gives it while it runs.  A request without a handle (waiting, or
preempted) has nothing computed, whatever its token list says: that is what makes
preemption by recomputation a matter of dropping the handle.

The field names the scheduler and callers read follow qwen3_runtime/engine/request.py:24-131
(``token_ids``, ``num_prompt_tokens``, ``num_scheduled_tokens``, ``max_tokens``,
``ignore_eos``, ``stop_token_ids``, ``min_tokens``, ``finish_reason``).
"""

from __future__ import annotations

import itertools
from enum import Enum, auto

import torch

from ..cache.manager import RequestCache
from ..sampling.params import SamplingParams


class RequestStatus(Enum):
    WAITING = auto()
    RUNNING = auto()
    FINISHED = auto()


_next_id = itertools.count()


def make_generator(seed: int | None) -> torch.Generator | None:
    """Seeded requests draw from a CPU generator of their own, so a seed gives the same
    uniforms whatever device the model is on (qwen3_runtime/sampling.py:293-298)."""
    if seed is None:
        return None
    return torch.Generator(device="cpu").manual_seed(int(seed))


class Request:
    def __init__(self, token_ids: list[int], max_tokens: int = 16, ignore_eos: bool = True, *,
                 sampling: SamplingParams | None = None, stop_token_ids: tuple[int, ...] = (),
                 min_tokens: int | None = None):
        if len(token_ids) == 0:
            raise ValueError("prompt token_ids must be non-empty")
        if max_tokens < 1:
            raise ValueError("max_tokens must be positive")
        self.request_id = next(_next_id)
        self.sampling = sampling if sampling is not None else SamplingParams()
        # tokens: the prompt, then everything sampled so far
        self.token_ids: list[int] = [int(t) for t in token_ids]
        self.num_prompt_tokens = len(self.token_ids)
        # limits and stops
        self.max_tokens = int(max_tokens)
        self.min_tokens = int(self.sampling.min_tokens if min_tokens is None else min_tokens)
        self.ignore_eos = bool(ignore_eos)
        self.stop_token_ids = tuple(int(t) for t in stop_token_ids)
        # progress
        self.status = RequestStatus.WAITING
        self.cache: RequestCache | None = None  # held only while running
        self.num_scheduled_tokens = 0  # its share of the step being put together or run
        self.num_preemptions = 0
        self.finish_reason: str | None = None
        # sampling state
        self.rng = make_generator(self.sampling.seed)
        self.logprobs: list[float] = []

    def __len__(self) -> int:
        return len(self.token_ids)

    @property
    def num_computed_tokens(self) -> int:
        """Tokens whose keys and values (or state) are in the cache."""
        return 0 if self.cache is None else self.cache.num_computed

    @property
    def uncomputed_tokens(self) -> int:
        """Known tokens not in the cache yet: the rest of the prompt, the token sampled last,
        or everything after a preemption."""
        return max(len(self.token_ids) - self.num_computed_tokens, 0)

    @property
    def is_prefill_complete(self) -> bool:
        return self.num_computed_tokens >= self.num_prompt_tokens

    @property
    def num_output_tokens(self) -> int:
        return len(self.token_ids) - self.num_prompt_tokens

    @property
    def output_token_ids(self) -> list[int]:
        return self.token_ids[self.num_prompt_tokens:]
