"""The engine: schedule, run the step function, sample, finish.

Parity: qwen3_runtime/engine/engine.py:53-92 (``add_request``), :216-260 (``step``),
:183-205 (``stream_request``), :359-366 (``generate``), :340-357 (per-step stats).
"""

from __future__ import annotations

from ..cache.manager import CacheManager
from ..config.engine_config import EngineConfig
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .batch import StepEntry
from .request import Request, RequestStatus
from .scheduler import Scheduler


class Engine:
    def __init__(self, config: EngineConfig, runner, cache: CacheManager, sampler: Sampler):
        self.config = config
        self.runner = runner
        self.cache = cache
        self.sampler = sampler
        self.scheduler = Scheduler(config, cache)
        self._requests: dict[int, Request] = {}
        self.last_step_stats: dict | None = None

    # ---- requests -----------------------------------------------------------------------
    def add_request(self, token_ids: list[int], max_tokens: int = 16, *, ignore_eos: bool = True,
                    sampling: SamplingParams | None = None, stop_token_ids: tuple[int, ...] = ()) -> int:
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
        preempt_before = self.scheduler.num_preemptions
        reqs = self.scheduler.schedule()
        if not reqs:
            self.last_step_stats = None
            return []
        entries, sampling = [], []
        for req in reqs:
            start = req.cache.num_computed
            end = start + req.num_scheduled_tokens
            samples = end >= len(req.token_ids)
            entries.append(StepEntry(req.cache, req.token_ids[start:end],
                                     [req.num_scheduled_tokens - 1] if samples else []))
            if samples:
                sampling.append(req)
        self.last_step_stats = self._collect_step_stats(reqs, preempt_before)
        logits = self.runner.run(entries)
        tokens: dict[int, int] = {}
        if sampling:
            # kernels with bounded waits report through a device word: its copy rides along with
            # the step and is looked at after the wait for the sampled tokens
            ops = self.sampler.ops
            if hasattr(ops, "watch_kernel_errors"):
                ops.watch_kernel_errors()
            toks, logprobs = self.sampler.sample(logits, sampling)
            if hasattr(ops, "raise_if_watched_error"):
                ops.raise_if_watched_error()
            for req, tok, lp in zip(sampling, toks, logprobs):
                tokens[req.request_id] = tok
                if lp is not None:
                    req.logprobs.append(lp)
        finished = {r.request_id for r in self.scheduler.postprocess(reqs, [tokens.get(r.request_id) for r in reqs])}
        out = [(r.request_id, tokens.get(r.request_id), r.request_id in finished) for r in reqs]
        for rid in finished:
            self._requests.pop(rid, None)
        return out

    def _collect_step_stats(self, reqs: list[Request], preempt_before: int) -> dict:
        stats = dict(req_ids=[r.request_id for r in reqs], prefill_tokens=0, decode_tokens=0, prefill_reqs=0,
                     decode_reqs=0, preempts=self.scheduler.num_preemptions - preempt_before)
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
