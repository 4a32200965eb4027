"""CUDA graphs for decode-only steps.

A step in which every request brings exactly one token launches a few hundred small
kernels; replaying them from a captured graph removes the launch cost.  One graph per
(batch-size bucket, block-table width bucket, what the parts' choosers answer for the
step's lengths): the batch is padded to the bucket with
dummy sequences that write to the cache's scratch page, the step's integer metadata is
copied into a fixed device buffer that the captured kernels read, and logits come out
of a fixed buffer.  Kernel choices inside a captured step depend on the key only: on the
buckets, and on the lengths of the moment only through the choosers' answers
(``Part.step_choosers``), e.g. the slice count of decode attention.
Parity: qwen3_runtime/engine/cuda_graph.py:79-249 (one graph per batch size, static
input and logits buffers, metadata refreshed outside the capture).
"""

from __future__ import annotations

import gc
from dataclasses import dataclass

import torch

from .batch import StepEntry


@dataclass
class _Captured:
    graph: torch.cuda.CUDAGraph
    meta: torch.Tensor  # fixed int32 device buffer with the step's metadata
    logits: torch.Tensor  # [bucket, vocab] float32, rewritten by every replay


def _bucket(n: int, sizes: list[int]) -> int | None:
    for s in sizes:
        if n <= s:
            return s
    return None


class DecodeGraphs:
    def __init__(self, runner, batch_sizes):
        self.runner = runner
        self.sizes = sorted(int(s) for s in batch_sizes)
        self.captured: dict[tuple, _Captured] = {}
        self.replays = 0
        # one memory pool for all captured steps: they never run at the same time (one stream), so
        # the buffers inside one may be the buffers inside another; only what a capture hands out
        # (its logits) stays its own
        self.pool = torch.cuda.graph_pool_handle() if torch.cuda.is_available() else None

    def try_run(self, entries: list[StepEntry], device_tokens: torch.Tensor | None = None) -> torch.Tensor | None:
        """Logits for the entries that want them (an empty tensor when none does), or None
        when the step is not a decode-only step that fits a bucket."""
        if any(len(e.tokens) != 1 for e in entries):
            return None
        B = len(entries)
        bucket = _bucket(B, self.sizes)
        if bucket is None:
            return None
        need = max((len(t) for e in entries for t in e.cache.tables), default=1)
        width = max(8, 1 << (max(need, 1) - 1).bit_length())
        # what the parts' kernels choose from the lengths of the moment is part of the key
        choices = self.runner.model.step_choices([e.cache.num_computed + 1 for e in entries])
        key = (bucket, width, tuple(sorted(choices.items())))
        cap = self.captured.get(key)
        if cap is None:
            cap = self._capture(key, choices)
        self._fill(cap, entries, bucket, width, need_context=False)
        if device_tokens is not None:  # ids that only the device knows, over the placeholders
            self.runner.builder.last_token_ids.copy_(device_tokens)
        cap.graph.replay()
        self.replays += 1
        wanted = [i for i, e in enumerate(entries) if e.want]
        if len(wanted) == B:
            return cap.logits[:B]
        if not wanted:
            return cap.logits[:0]
        return cap.logits[torch.tensor(wanted, dtype=torch.long, device=cap.logits.device)]

    def _fill(self, cap: _Captured, entries, bucket: int, width: int, need_context: bool = True):
        r = self.runner
        return r.builder.build(entries, pad_to=bucket, table_width=width, scratch_page=r.storage.scratch_page,
                               scratch_slot=r.storage.scratch_slot, device_buffer=cap.meta, all_rows=True,
                               need_context=need_context)

    def _capture(self, key, choices: dict) -> _Captured:
        """Warm up and capture a step made of padding rows only: every row reads and writes the
        scratch page and the scratch state slot, so neither the warm-up run nor the capture
        touches a live request's keys, values or state (a state layer advanced by the warm-up
        and again by the first replay would count that token twice).  The real step's metadata
        is copied into ``meta`` afterwards, by :meth:`try_run`, and only then replayed."""
        bucket, width = key[:2]
        r = self.runner
        n_paged = len(r.cache.paged_groups)
        meta = torch.zeros(8 * bucket + 64 + n_paged * bucket * width, dtype=torch.int32, device=r.device)
        cap = _Captured(torch.cuda.CUDAGraph(), meta, None)
        step = self._fill(cap, [], bucket, width)
        step.captured_width = width
        step.choices = dict(choices)
        # warm up on a side stream (loads kernels, builds shared tables), then capture
        side = torch.cuda.Stream(device=r.device)
        side.wait_stream(torch.cuda.current_stream(r.device))
        with torch.cuda.stream(side):
            r.model.forward(step, r.storage)
        torch.cuda.current_stream(r.device).wait_stream(side)
        torch.cuda.synchronize(r.device)
        # Python's cycle collector must not run inside the capture: if it finds a dead engine
        # there (engines hold cycles), freeing its graphs, pinned buffers and events makes CUDA
        # calls that are not allowed while a stream is capturing and invalidates the capture.
        gc.collect()
        was_enabled = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(cap.graph, pool=self.pool):
                cap.logits = r.model.forward(step, r.storage)
        finally:
            if was_enabled:
                gc.enable()
        self.captured[key] = cap
        return cap
