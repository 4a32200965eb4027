"""The step function.

``ModelRunner.run(entries)`` takes a batch of (request, its next tokens, wanted
places) -- portions of prompts beside single decoded tokens, cut anywhere -- runs
exactly those tokens as one batch against the cache that earlier steps left, stores
their keys and values, and returns float32 logits at the wanted places, in the order
of the entries and of each entry's ``want``.  It samples nothing: the engine samples
from what it returns, and trace replay writes it to disk.
Parity: qwen3_runtime/engine/model_runner.py:107-192 (``run`` / ``run_logits`` /
``_run_group``); there is no prefill/decode split here, one launch sequence serves
every mix.
"""

from __future__ import annotations

import torch

from ..cache.manager import CacheManager
from ..cache.storage import CacheStorage
from ..parts.model import DecoderModel
from .batch import BatchBuilder, StepEntry


class ModelRunner:
    def __init__(self, model: DecoderModel, cache: CacheManager, storage: CacheStorage, *,
                 max_positions: int, cuda_graph: bool = False, graph_batch_sizes=(1, 2, 4, 8, 16, 32, 64)):
        self.model = model
        self.cache = cache
        self.storage = storage
        self.device = model.ctx.device
        self.builder = BatchBuilder(cache, self.device, vocab_size=model.spec.vocab_size,
                                    max_positions=max_positions)
        self.graphs = None
        if cuda_graph:
            from .graph import DecodeGraphs

            self.graphs = DecodeGraphs(self, graph_batch_sizes)
        self.num_steps = 0

    def run(self, entries: list[StepEntry], device_tokens: torch.Tensor | None = None) -> torch.Tensor | None:
        """One step; returns logits ``[sum(len(want)), vocab]`` float32, or None.

        ``device_tokens`` (int32, one per entry, every entry bringing one token): the token ids
        are on the device only -- sampled by a step whose result the host has not read yet --
        and replace the placeholders in ``entries`` after the step's metadata is packed."""
        if device_tokens is not None and (any(len(e.tokens) != 1 for e in entries)
                                          or device_tokens.numel() != len(entries)):
            raise ValueError("device_tokens: one token per entry, every entry bringing exactly one")
        resets = [e.cache.slot for e in entries if e.cache.needs_state_reset]
        if resets:
            self.storage.zero_state_slots(resets)
            for e in entries:
                e.cache.needs_state_reset = False
        logits = None
        if self.graphs is not None:
            logits = self.graphs.try_run(entries, device_tokens)
        if logits is None:
            step = self.builder.build(entries, scratch_page=self.storage.scratch_page,
                                      scratch_slot=self.storage.scratch_slot)
            if device_tokens is not None:
                self.builder.last_token_ids.copy_(device_tokens)
            if step.decode_only:
                step.choices = self.model.step_choices(step.host_kv_lens)
            logits = self.model.forward(step, self.storage)
        else:
            logits = logits if logits.numel() else None
        for e in entries:
            self.cache.commit(e.cache, len(e.tokens))
        self.num_steps += 1
        return logits
