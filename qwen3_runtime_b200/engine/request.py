"""One request: token ids, progress, sampling state and stop conditions.

Parity: qwen3_runtime/engine/request.py:24-131 (fields and counters that the
scheduler reads); what the reference keeps for sessions, prefix cache, speculative
drafts and offload has no counterpart here.
"""

from __future__ import annotations

from enum import Enum, auto
from itertools import count

import torch

from ..cache.manager import RequestCache
from ..sampling.params import SamplingParams


class RequestStatus(Enum):
    WAITING = auto()
    RUNNING = auto()
    FINISHED = auto()


class Request:
    _ids = count()

    def __init__(self, token_ids: list[int], max_tokens: int = 16, ignore_eos: bool = True, *,
                 sampling: SamplingParams | None = None, stop_token_ids: tuple[int, ...] = (),
                 min_tokens: int | None = None):
        if not token_ids:
            raise ValueError("prompt token_ids must be non-empty")
        if max_tokens < 1:
            raise ValueError("max_tokens must be positive")
        self.request_id = next(Request._ids)
        self.status = RequestStatus.WAITING
        self.token_ids = [int(t) for t in token_ids]
        self.num_prompt_tokens = len(self.token_ids)
        self.num_scheduled_tokens = 0
        self.max_tokens = max_tokens
        self.ignore_eos = ignore_eos
        self.sampling = sampling or SamplingParams()
        self.stop_token_ids = tuple(stop_token_ids)
        self.min_tokens = int(self.sampling.min_tokens if min_tokens is None else min_tokens)
        self.rng = make_generator(self.sampling.seed)
        self.cache: RequestCache | None = None  # open while the request is running
        self.logprobs: list[float] = []
        self.finish_reason: str | None = None
        self.num_preemptions = 0

    def __len__(self) -> int:
        return len(self.token_ids)

    @property
    def num_computed_tokens(self) -> int:
        return self.cache.num_computed if self.cache is not None else 0

    @property
    def uncomputed_tokens(self) -> int:
        """Tokens of ``token_ids`` not in the cache yet (prompt, or recompute after preemption)."""
        return max(0, len(self.token_ids) - self.num_computed_tokens)

    @property
    def is_prefill_complete(self) -> bool:
        return self.num_computed_tokens >= self.num_prompt_tokens

    @property
    def num_output_tokens(self) -> int:
        return len(self.token_ids) - self.num_prompt_tokens

    @property
    def output_token_ids(self) -> list[int]:
        return self.token_ids[self.num_prompt_tokens:]


def make_generator(seed: int | None) -> torch.Generator | None:
    """A CPU generator per seeded request, so a seed means the same draws on every
    device (qwen3_runtime/sampling.py:293-298)."""
    if seed is None:
        return None
    gen = torch.Generator(device="cpu")
    gen.manual_seed(int(seed))
    return gen
