"""Who runs in the next step, and with how many tokens.

A step has two scarce things: *tokens* (``max_num_batched_tokens``) and *seats*
(``max_num_seqs``).  :meth:`Scheduler.schedule` hands them out in two passes over
its queues -- requests that already hold pages first, in the order they were
admitted, then newcomers in arrival order -- and each grant is trimmed to what the
cache manager can still reserve for that request in *every* cache group (pages of
a full-attention group, pages of a window group, its state slot).  A grant of one
token is a decode step for that request; a larger one is a portion of a prompt, or
of a recomputation.

When the pass grants nothing although requests hold pages, the pool is exhausted.
The answer is *preemption by recomputation*: the request admitted last gives back
all pages and its slot and returns to the head of the arrival queue with every
token it has (prompt and generated); it is computed again from its first token and
samples only after it has caught up.  A newcomer that finds no room in an
otherwise idle pool can never run, and says so.

Behaviour kept from qwen3_runtime/engine/scheduler.py:34-122, 227-314 (running before
waiting, FCFS with head-of-line blocking by a long prompt, youngest preempted first,
finish on stop token / EOS after ``min_tokens`` / ``max_tokens``).
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

from ..cache.manager import CacheManager
from ..config.engine_config import EngineConfig
from .request import Request, RequestStatus


@dataclass
class _StepPlan:
    """What one scheduling pass has handed out so far."""

    tokens_left: int
    seats_left: int
    granted: list[Request] = field(default_factory=list)

    @property
    def open(self) -> bool:
        return self.tokens_left > 0 and self.seats_left > 0

    def grant(self, req: Request, n: int) -> None:
        req.num_scheduled_tokens = n
        self.granted.append(req)
        self.tokens_left -= n
        self.seats_left -= 1


class Scheduler:
    def __init__(self, config: EngineConfig, cache: CacheManager):
        self.config = config
        self.cache = cache
        self.waiting: deque[Request] = deque()  # arrival order; preempted requests re-enter at the head
        self.running: deque[Request] = deque()  # admission order: the last one is the youngest
        self.num_preemptions = 0

    # ---- arrivals and departures ------------------------------------------------------------
    def add(self, req: Request) -> None:
        """Queue a request.  One whose prompt and output together could not be held even by an
        empty pool is refused here rather than left to starve."""
        longest = len(req.token_ids) + req.max_tokens
        if not self.cache.fits_at_all(longest):
            raise RuntimeError(f"request length {longest} needs {self.cache.pages_for(longest)} KV blocks; "
                               f"pool has {min(self.cache.num_pages)}")
        req.status = RequestStatus.WAITING
        self.waiting.append(req)

    def abort(self, req: Request) -> None:
        """Take a request out wherever it is and give back what it holds."""
        if req in self.waiting:
            self.waiting.remove(req)
        if req.status is not RequestStatus.FINISHED:
            req.finish_reason = req.finish_reason or "abort"
            self._retire(req)

    def is_finished(self) -> bool:
        return not (self.waiting or self.running)

    # ---- one step's batch ---------------------------------------------------------------------
    def schedule(self) -> list[Request]:
        """The requests of the next step, each with ``num_scheduled_tokens`` set and pages
        reserved for exactly those tokens.  Empty when there is nothing to do."""
        # every failed pass evicts one running request, so the number of passes is bounded
        for _ in range(len(self.running) + 1):
            plan = _StepPlan(self.config.max_num_batched_tokens, self.config.max_num_seqs)
            self._serve_running(plan)
            self._admit_waiting(plan)
            if plan.granted:
                return plan.granted
            if not self.running:
                break
            self._evict(self.running[-1])
        if self.waiting:
            raise RuntimeError("waiting request exceeds the KV pool even after shrinking the chunk")
        return []

    def _grantable(self, req: Request, plan: _StepPlan) -> int:
        """Tokens of ``req`` this pass can take: what it still has to compute, within the tokens
        left, trimmed to what every cache group can reserve for it right now."""
        want = min(req.uncomputed_tokens, plan.tokens_left)
        return self.cache.max_reservable(req.cache, want) if want > 0 else 0

    def _serve_running(self, plan: _StepPlan) -> None:
        for req in self.running:
            if not plan.open:
                return
            n = self._grantable(req, plan)
            if n > 0:
                self.cache.reserve(req.cache, n)
                plan.grant(req, n)

    def _admit_waiting(self, plan: _StepPlan) -> None:
        """Newcomers in arrival order.  One that gets nothing this pass keeps its place in the
        queue; the ones behind it are still looked at (they may be shorter)."""
        passed_over: list[Request] = []
        while self.waiting and plan.open and self.cache.slots.num_free > 0:
            req = self.waiting.popleft()
            req.cache = self.cache.open(req.request_id)
            n = self._grantable(req, plan)
            if n <= 0:
                self.cache.close(req.cache)
                req.cache = None
                passed_over.append(req)
                continue
            self.cache.reserve(req.cache, n)
            req.status = RequestStatus.RUNNING
            self.running.append(req)
            plan.grant(req, n)
        self.waiting.extendleft(reversed(passed_over))

    def _evict(self, req: Request) -> None:
        """Preempt: everything ``req`` holds goes back to the pool; its tokens stay with it."""
        self.running.remove(req)
        self.cache.close(req.cache)
        req.cache = None
        req.num_scheduled_tokens = 0
        req.status = RequestStatus.WAITING
        req.num_preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(req)

    # ---- after the step ran ---------------------------------------------------------------------
    def postprocess(self, reqs: list[Request], token_ids: list[int | None]) -> list[Request]:
        """Take the step's sampled tokens (``None`` for a request whose portion ended before its
        last known token) and retire the requests that are done; returns those.  The step
        function has already counted the portion as computed."""
        if len(token_ids) != len(reqs):
            raise ValueError("token_ids must align with scheduled requests")
        done = []
        for req, tok in zip(reqs, token_ids):
            req.num_scheduled_tokens = 0
            if tok is None:
                continue
            req.token_ids.append(int(tok))
            req.finish_reason = self._why_done(req, int(tok))
            if req.finish_reason is not None:
                self._retire(req)
                done.append(req)
        return done

    def _why_done(self, req: Request, token: int) -> str | None:
        produced = req.num_output_tokens
        if not req.ignore_eos and produced >= req.min_tokens:
            if token in req.stop_token_ids or token == self.config.eos_token_id:
                return "stop"
        return "length" if produced >= req.max_tokens else None

    def _retire(self, req: Request) -> None:
        req.status = RequestStatus.FINISHED
        if req.cache is not None:
            self.cache.close(req.cache)
            req.cache = None
        if req in self.running:
            self.running.remove(req)
