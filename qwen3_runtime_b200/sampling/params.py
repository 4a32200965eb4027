"""Sampling hyper-parameters, with the reference's names and meanings.

Parity: qwen3_runtime/sampling_params.py:9-46.  ``temperature <= 0`` is greedy.
The chain is: logit_bias -> penalties -> (greedy stops here) -> / temperature ->
min_p -> top_k -> top_p -> softmax -> inverse-CDF draw.
"""

from __future__ import annotations

import math
from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    min_p: float = 0.0
    seed: int | None = None
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    logit_bias: dict[int, float] | None = None
    min_tokens: int = 0
    logprobs: bool = False

    def __post_init__(self) -> None:
        # the same values are refused as in qwen3_runtime/sampling_params.py:31-46
        problems = []
        for name in ("temperature", "top_p", "min_p", "repetition_penalty", "presence_penalty",
                     "frequency_penalty"):
            if not math.isfinite(getattr(self, name)):
                problems.append(f"{name} must be finite")
        if not problems:
            if not 0.0 < self.top_p <= 1.0:
                problems.append("top_p must satisfy 0 < top_p <= 1")
            if not 0.0 <= self.min_p <= 1.0:
                problems.append("min_p must satisfy 0 <= min_p <= 1")
            if self.repetition_penalty <= 0.0:
                problems.append("repetition_penalty must be positive and finite")
        if self.min_tokens < 0:
            problems.append("min_tokens must be non-negative")
        if problems:
            raise ValueError("invalid sampling parameters: " + "; ".join(problems))

    def is_greedy(self) -> bool:
        return self.temperature <= 0.0

    def has_penalties(self) -> bool:
        return not (
            self.repetition_penalty == 1.0 and self.presence_penalty == 0.0 and self.frequency_penalty == 0.0
        )

    def needs_filter(self) -> bool:
        """True when the draw needs more than softmax(logits / temperature)."""
        return self.min_p > 0.0 or self.top_k > 0 or self.top_p < 1.0
