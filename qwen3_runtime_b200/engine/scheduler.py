"""Continuous batching with chunked prefill and preemption by recompute.

Every ``schedule()`` call spends a token budget (``max_num_batched_tokens``): first on
the running requests in admission order (a decoding request needs one token, a request
still in its prompt as much as is left), then on waiting requests, first come first
served, while fewer than ``max_num_seqs`` requests are scheduled.  A portion is shrunk
to the pages that are free; pages are reserved only for the tokens scheduled.

When pages run out -- nothing at all could be scheduled although requests are running
-- the youngest running request is preempted: its pages and state slot are returned,
it goes to the front of the waiting queue with all its tokens (prompt and generated),
and is later prefilled again from its first token; it samples again only once it has
caught up.  A waiting request that can never fit raises.
Parity: qwen3_runtime/engine/scheduler.py:34-122, 227-314.
"""

from __future__ import annotations

from collections import deque

from ..cache.manager import CacheManager
from ..config.engine_config import EngineConfig
from .request import Request, RequestStatus


class Scheduler:
    def __init__(self, config: EngineConfig, cache: CacheManager):
        self.config = config
        self.cache = cache
        self.waiting: deque[Request] = deque()
        self.running: deque[Request] = deque()
        self.num_preemptions = 0

    # ---- admission --------------------------------------------------------------------
    def add(self, req: Request) -> None:
        max_len = len(req.token_ids) + req.max_tokens
        if not self.cache.fits_at_all(max_len):
            raise RuntimeError(
                f"request length {max_len} needs {self.cache.pages_for(max_len)} KV blocks; "
                f"pool has {min(self.cache.num_pages)}")
        req.status = RequestStatus.WAITING
        self.waiting.append(req)

    def is_finished(self) -> bool:
        return not self.waiting and not self.running

    # ---- one step's batch ---------------------------------------------------------------
    def schedule(self) -> list[Request]:
        bound = self.config.max_num_seqs + len(self.running) + len(self.waiting) + 1
        for _ in range(max(bound, 1)):
            scheduled: list[Request] = []
            budget = self._schedule_running(scheduled, self.config.max_num_batched_tokens)
            self._schedule_waiting(scheduled, budget)
            if scheduled:
                return scheduled
            if self.running:
                self._preempt(self.running.pop())
                continue
            if self.waiting:
                raise RuntimeError("waiting request exceeds the KV pool even after shrinking the chunk")
            return []
        raise RuntimeError("scheduler could not admit a batch after preemption")

    def _tokens_to_schedule(self, req: Request, budget: int) -> int:
        remaining = req.uncomputed_tokens
        if remaining <= 0 or budget <= 0:
            return 0
        return self.cache.max_reservable(req.cache, min(remaining, budget))

    def _schedule_running(self, scheduled: list[Request], budget: int) -> int:
        for req in self.running:
            if len(scheduled) >= self.config.max_num_seqs or budget <= 0:
                continue
            n = self._tokens_to_schedule(req, budget)
            if n <= 0:
                continue
            self.cache.reserve(req.cache, n)
            req.num_scheduled_tokens = n
            scheduled.append(req)
            budget -= n
        return budget

    def _schedule_waiting(self, scheduled: list[Request], budget: int) -> None:
        deferred: deque[Request] = deque()
        while self.waiting:
            if len(scheduled) >= self.config.max_num_seqs or budget <= 0:
                break
            if self.cache.slots.num_free == 0:
                break
            req = self.waiting.popleft()
            req.cache = self.cache.open(req.request_id)
            n = self._tokens_to_schedule(req, budget)
            if n <= 0:
                self.cache.close(req.cache)
                req.cache = None
                deferred.append(req)
                continue
            self.cache.reserve(req.cache, n)
            req.num_scheduled_tokens = n
            req.status = RequestStatus.RUNNING
            scheduled.append(req)
            self.running.append(req)
            budget -= n
        self.waiting.extendleft(reversed(deferred))

    def _preempt(self, req: Request) -> None:
        self.cache.close(req.cache)
        req.cache = None
        req.num_scheduled_tokens = 0
        req.status = RequestStatus.WAITING
        req.num_preemptions += 1
        self.waiting.appendleft(req)
        self.num_preemptions += 1

    # ---- after the forward ----------------------------------------------------------------
    def postprocess(self, reqs: list[Request], token_ids: list[int | None]) -> list[Request]:
        """Append sampled tokens (``None``: the request's portion did not reach the end of
        its known tokens) and finish what is done.  The runner has already advanced
        each request's computed count."""
        if len(token_ids) != len(reqs):
            raise ValueError("token_ids must align with scheduled requests")
        finished = []
        for req, tok in zip(reqs, token_ids):
            req.num_scheduled_tokens = 0
            if tok is None:
                continue
            req.token_ids.append(int(tok))
            reason = self._finish_reason(req, int(tok))
            if reason is not None:
                req.finish_reason = reason
                self._finish(req)
                finished.append(req)
        return finished

    def _finish_reason(self, req: Request, token_id: int) -> str | None:
        n_out = req.num_output_tokens
        hit_stop = (not req.ignore_eos) and (
            token_id in req.stop_token_ids
            or (self.config.eos_token_id is not None and token_id == self.config.eos_token_id))
        if hit_stop and n_out >= req.min_tokens:
            return "stop"
        if n_out >= req.max_tokens:
            return "length"
        return None

    def _finish(self, req: Request) -> None:
        req.status = RequestStatus.FINISHED
        if req.cache is not None:
            self.cache.close(req.cache)
            req.cache = None
        try:
            self.running.remove(req)
        except ValueError:
            pass

    def abort(self, req: Request) -> None:
        """Drop a request from every queue and return what it holds."""
        try:
            self.waiting.remove(req)
        except ValueError:
            pass
        if req.status != RequestStatus.FINISHED:
            req.finish_reason = req.finish_reason or "abort"
            self._finish(req)
