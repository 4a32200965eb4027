"""The engine: schedule, run the step function, sample, finish.

Parity: qwen3_runtime/engine/engine.py:53-92 (``add_request``), :216-260 (``step``),
:183-205 (``stream_request``), :359-366 (``generate``), :340-357 (per-step stats).

Running ahead.  A decode step's only input that the host does not know beforehand is the
token the step before it sampled, and that token is on the device already.  So while the
requests just keep decoding, ``step()`` puts the next step on the device (its token ids
copied from the sampler's output, device to device) *before* it waits for the tokens of the
step it returns; the device then never waits for the host between steps.  What the host
cannot know in time is a stop token: if a request turns out to have finished, the step that
was already running for it is simply not read for that request (its pages were returned when
it finished; work queued later on the same stream comes after the abandoned writes).  Nothing
runs ahead when the batch is about to change: a request waits for admission, one reaches its
``max_tokens``, pages may run out, or a request's sampling needs the token history on the
host (penalties).  Every request gets the same tokens with and without running ahead; a request
that is added while a step is already running ahead joins one step later than it would otherwise.
"""

from __future__ import annotations

from ..cache.manager import CacheManager
from ..config.engine_config import EngineConfig
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .batch import StepEntry
from .request import Request, RequestStatus
from .scheduler import Scheduler


class _Launched:
    """A step that is on the device: who takes part, who samples, and the sampler's handle."""

    __slots__ = ("reqs", "sampling", "sampled", "decode_only", "stats")

    def __init__(self, reqs, sampling, sampled, decode_only, stats):
        self.reqs, self.sampling, self.sampled = reqs, sampling, sampled
        self.decode_only, self.stats = decode_only, stats


class Engine:
    def __init__(self, config: EngineConfig, runner, cache: CacheManager, sampler: Sampler):
        self.config = config
        self.runner = runner
        self.cache = cache
        self.sampler = sampler
        self.scheduler = Scheduler(config, cache)
        self._requests: dict[int, Request] = {}
        self.last_step_stats: dict | None = None
        self._ahead: _Launched | None = None  # the step launched before the last one was read
        self.num_run_ahead = 0

    # ---- requests -----------------------------------------------------------------------
    def add_request(self, token_ids: list[int], max_tokens: int = 16, *, ignore_eos: bool = True,
                    sampling: SamplingParams | None = None, stop_token_ids: tuple[int, ...] = ()) -> int:
        """Queue a request.  Refused here, before it can take part in a step: token ids outside
        the vocabulary, and a prompt that leaves no room for a single new token within the
        positions the model serves.  ``max_tokens`` is cut to the positions that are left, so
        such a request ends with ``length`` at the limit instead of failing in a later step."""
        builder = getattr(self.runner, "builder", None)
        if builder is not None:
            vocab, limit = builder.vocab_size, builder.max_positions
            bad = next((int(t) for t in token_ids if not 0 <= int(t) < vocab), None)
            if bad is not None:
                raise ValueError(f"token id {bad} is outside the vocabulary of {vocab}")
            # the last sampled token is never fed back, so prompt + max_tokens - 1 positions are used
            if len(token_ids) > limit:
                raise ValueError(f"a prompt of {len(token_ids)} tokens leaves no room for a new token: the "
                                 f"model's position encoding covers {limit} positions")
            max_tokens = min(max_tokens, limit - len(token_ids) + 1)
        req = Request(token_ids, max_tokens=max_tokens, ignore_eos=ignore_eos, sampling=sampling,
                      stop_token_ids=stop_token_ids)
        self.scheduler.add(req)
        self._requests[req.request_id] = req
        return req.request_id

    def get_request(self, request_id: int) -> Request:
        return self._requests[request_id]

    def abort_request(self, request_id: int) -> None:
        req = self._requests.pop(request_id, None)
        if req is not None:
            self.scheduler.abort(req)

    def is_finished(self) -> bool:
        return self.scheduler.is_finished()

    # ---- one step -------------------------------------------------------------------------
    def step(self) -> list[tuple[int, int | None, bool]]:
        """Schedule and run one batch.  Returns ``(request_id, new token or None, finished)``
        for every request that took part."""
        launched, self._ahead = self._ahead, None
        if launched is not None and all(r.status == RequestStatus.FINISHED for r in launched.reqs):
            launched = None  # everyone it ran for has finished or was aborted meanwhile
        if launched is None:
            preempt_before = self.scheduler.num_preemptions
            reqs = self.scheduler.schedule()
            if not reqs:
                self.last_step_stats = None
                return []
            launched = self._launch(reqs, preempt_before)
        self.last_step_stats = launched.stats
        failure = None
        if self.config.run_ahead and self._may_run_ahead(launched):
            try:
                self._ahead = self._launch_next_decode(launched)
            except Exception as exc:  # noqa: BLE001 - re-raised below, after this step was read
                # the step that is on the device is still read, so that its tokens are not lost
                # and every request's counters stay consistent with its cache
                self._ahead, failure = None, exc
        out = self._read(launched)
        if failure is not None:
            raise failure
        return out

    def _launch(self, reqs: list[Request], preempt_before: int) -> _Launched:
        entries, sampling = [], []
        for req in reqs:
            start = req.cache.num_computed
            end = start + req.num_scheduled_tokens
            samples = end >= len(req.token_ids)
            entries.append(StepEntry(req.cache, req.token_ids[start:end],
                                     [req.num_scheduled_tokens - 1] if samples else []))
            if samples:
                sampling.append(req)
        stats = self._collect_step_stats(reqs, preempt_before)
        decode_only = len(sampling) == len(reqs) and all(r.num_scheduled_tokens == 1 for r in reqs)
        logits = self.runner.run(entries)
        return _Launched(reqs, sampling, self._sample(logits, sampling), decode_only, stats)

    def _sample(self, logits, sampling: list[Request]):
        if not sampling:
            return None
        # kernels with bounded waits report through a device word: its copy rides along with
        # the step and is looked at after the wait for the sampled tokens
        ops = self.sampler.ops
        if hasattr(ops, "watch_kernel_errors"):
            ops.watch_kernel_errors()
        return self.sampler.launch(logits, sampling)

    def _may_run_ahead(self, launched: _Launched) -> bool:
        """The next step is this one again, one token further, whatever this one samples --
        unless a stop token ends a request, which is found out afterwards."""
        if not launched.decode_only or self.scheduler.waiting:
            return False
        reqs = launched.reqs
        if len(reqs) != len(self.scheduler.running) or any(a is not b for a, b in zip(reqs, self.scheduler.running)):
            return False
        for r in reqs:
            # the token on its way is output number num_output_tokens + 1: the last one allowed?
            if r.status != RequestStatus.RUNNING or r.num_output_tokens + 1 >= r.max_tokens:
                return False
            if r.sampling.has_penalties():  # needs the token on its way in the host's history
                return False
        # pages for everybody's next token, without preempting anyone
        free = list(self.cache.num_free_pages)
        for r in reqs:
            for g, n in enumerate(self.cache.new_pages_needed(r.cache, 1)):
                free[g] -= n
        return all(f >= 0 for f in free)

    def _launch_next_decode(self, before: _Launched) -> _Launched:
        reqs = before.reqs
        entries = []
        for req in reqs:
            self.cache.reserve(req.cache, 1)
            req.num_scheduled_tokens = 1
            entries.append(StepEntry(req.cache, [0], [0]))  # the id is on the device: before.sampled.tokens
        stats = self._collect_step_stats(reqs, self.scheduler.num_preemptions)
        logits = self.runner.run(entries, device_tokens=before.sampled.tokens)
        self.num_run_ahead += 1
        return _Launched(reqs, list(reqs), self._sample(logits, reqs), True, stats)

    def _read(self, launched: _Launched) -> list[tuple[int, int | None, bool]]:
        """Wait for the step's tokens, append them, finish what is done."""
        tokens: dict[int, int] = {}
        if launched.sampled is not None:
            toks, logprobs = self.sampler.read(launched.sampled)
            ops = self.sampler.ops
            if hasattr(ops, "raise_if_watched_error"):
                ops.raise_if_watched_error()
            for req, tok, lp in zip(launched.sampling, toks, logprobs):
                tokens[req.request_id] = tok
                if lp is not None and req.status != RequestStatus.FINISHED:
                    req.logprobs.append(lp)
        # a request that finished while this step was already running for it takes no part
        reqs = [r for r in launched.reqs if r.status != RequestStatus.FINISHED]
        finished = {r.request_id for r in self.scheduler.postprocess(reqs, [tokens.get(r.request_id) for r in reqs])}
        out = [(r.request_id, tokens.get(r.request_id), r.request_id in finished) for r in reqs]
        for rid in finished:
            self._requests.pop(rid, None)
        return out

    def _collect_step_stats(self, reqs: list[Request], preempt_before: int) -> dict:
        stats = dict(req_ids=[r.request_id for r in reqs], prefill_tokens=0, decode_tokens=0, prefill_reqs=0,
                     decode_reqs=0, preempts=self.scheduler.num_preemptions - preempt_before,
                     # per request: (tokens already in the cache, tokens this step runs)
                     spans=[(r.num_computed_tokens, r.num_scheduled_tokens) for r in reqs])
        for r in reqs:
            kind = "decode" if r.is_prefill_complete else "prefill"
            stats[kind + "_tokens"] += r.num_scheduled_tokens
            stats[kind + "_reqs"] += 1
        return stats

    # ---- whole requests -------------------------------------------------------------------
    def stream_request(self, request_id: int):
        """Yield the request's new token ids until it finishes (other live requests advance too)."""
        req = self._requests[request_id]
        while req.status != RequestStatus.FINISHED:
            progressed = False
            for rid, tok, _done in self.step():
                progressed = True
                if rid == request_id and tok is not None:
                    yield tok
            if not progressed:
                raise RuntimeError(f"request {request_id} status={req.status.name} made no progress")

    def generate(self, token_ids: list[int], max_tokens: int = 16, **kwargs) -> list[int]:
        return list(self.stream_request(self.add_request(token_ids, max_tokens=max_tokens, **kwargs)))

    def generate_batch(self, prompts: list[list[int]], max_tokens: int = 16, *,
                       sampling: SamplingParams | list[SamplingParams] | None = None, **kwargs) -> list[list[int]]:
        """Run several requests together under the scheduler; outputs in the order given."""
        if isinstance(sampling, (list, tuple)):
            if len(sampling) != len(prompts):
                raise ValueError("one SamplingParams per prompt, or a single one for all")
            per = list(sampling)
        else:
            per = [sampling] * len(prompts)
        reqs = [self._requests[self.add_request(p, max_tokens=max_tokens, sampling=s, **kwargs)]
                for p, s in zip(prompts, per)]
        while any(r.status != RequestStatus.FINISHED for r in reqs):
            if not self.step():
                raise RuntimeError("engine made no progress while requests remain")
        return [r.output_token_ids for r in reqs]

    def config_report(self) -> dict[str, object]:
        cfg = self.config
        return {
            "block_size": cfg.block_size,
            "num_kv_blocks": self.cache.num_pages,
            "max_num_seqs": cfg.max_num_seqs,
            "max_num_batched_tokens": cfg.max_num_batched_tokens,
            "cuda_graph": cfg.cuda_graph,
            "dtype": cfg.dtype,
            "eos_token_id": cfg.eos_token_id,
        }
