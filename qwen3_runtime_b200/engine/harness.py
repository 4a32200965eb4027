"""Closed-batch runs through an engine's public API, with per-request and per-step records.

``run_closed_batch`` submits every prompt at time zero and steps the engine until all
are finished, noting when each token of each request arrived (time to first token, time
per output token) and what every step was made of.  It works with any engine that has
``add_request(token_ids, max_tokens=, ignore_eos=)``, ``step() -> [(request_id, token or
None, finished)]`` and ``is_finished()``, which is this engine's API and the reference's
(qwen3_runtime/serving/slo_harness.py:390-416 is the reference's loop of the same name;
bench/metrics.py:69-163 its summary: median TTFT / TPOT over requests, output tokens per
second over the wall time of the run).
"""

from __future__ import annotations

import statistics
import time
from dataclasses import dataclass, field


@dataclass
class RequestTrace:
    request_id: int
    prompt_len: int
    max_tokens: int
    arrival_s: float
    token_times: list[float] = field(default_factory=list)

    @property
    def ttft_s(self) -> float | None:
        return self.token_times[0] - self.arrival_s if self.token_times else None

    @property
    def tpot_s(self) -> float | None:
        n = len(self.token_times)
        return (self.token_times[-1] - self.token_times[0]) / (n - 1) if n > 1 else None


@dataclass
class StepRecord:
    seconds: float  # wall time from the previous step's return to this one's
    prefill_tokens: int
    decode_tokens: int
    spans: list[tuple[int, int]]  # per request of the step: (tokens already in the cache, tokens run)
    preempts: int = 0

    @property
    def kind(self) -> str:
        if self.prefill_tokens and self.decode_tokens:
            return "mixed"
        return "prefill" if self.prefill_tokens else "decode"


def run_closed_batch(engine, prompts: list[list[int]], max_tokens: int | list[int], *, ignore_eos: bool = True,
                     synchronize=None, **request_kwargs) -> tuple[list[RequestTrace], list[StepRecord], float]:
    """All ``prompts`` arrive at once; returns ``(traces, step records, wall seconds)``.
    ``synchronize``: called before the clock starts and after the last step (a device
    synchronisation, so that the wall time covers all device work)."""
    lengths = list(max_tokens) if isinstance(max_tokens, (list, tuple)) else [int(max_tokens)] * len(prompts)
    if synchronize is not None:
        synchronize()
    t0 = time.perf_counter()
    traces: dict[int, RequestTrace] = {}
    for prompt, n_out in zip(prompts, lengths):
        rid = engine.add_request(prompt, max_tokens=n_out, ignore_eos=ignore_eos, **request_kwargs)
        traces[rid] = RequestTrace(rid, len(prompt), n_out, t0)
    records: list[StepRecord] = []
    last = t0
    while not engine.is_finished():
        out = engine.step()
        now = time.perf_counter()
        for rid, tok, _finished in out:
            if tok is not None and rid in traces:
                traces[rid].token_times.append(now)
        stats = getattr(engine, "last_step_stats", None)
        if stats is not None:
            records.append(StepRecord(now - last, stats.get("prefill_tokens", 0), stats.get("decode_tokens", 0),
                                      list(stats.get("spans", ())), stats.get("preempts", 0)))
        last = now
        if not out and not engine.is_finished():
            raise RuntimeError("the engine made no progress while requests remain")
    if synchronize is not None:
        synchronize()
    return list(traces.values()), records, time.perf_counter() - t0


def _spread(xs: list[float]) -> dict:
    if not xs:
        return dict(median=None, mean=None, min=None, max=None)
    return dict(median=statistics.median(xs), mean=statistics.fmean(xs), min=min(xs), max=max(xs))


def summarize(traces: list[RequestTrace], wall_s: float) -> dict:
    """Output tokens per second over the run, and TTFT / TPOT over its requests."""
    n_out = sum(len(t.token_times) for t in traces)
    return dict(
        n_requests=len(traces),
        forced_length_ok=all(len(t.token_times) == t.max_tokens for t in traces),
        output_tokens=n_out,
        output_tok_s=n_out / wall_s if wall_s > 0 else 0.0,
        ttft_s=_spread([t.ttft_s for t in traces if t.ttft_s is not None]),
        tpot_s=_spread([t.tpot_s for t in traces if t.tpot_s is not None]),
        wall_s=wall_s,
    )


@dataclass
class ModelCost:
    """What a step of a dense decoder has to read and compute, from the model's sizes."""

    weight_bytes: float  # every weight a step uses, once
    kv_bytes_per_token: float  # keys and values of one cached token, all layers
    linear_flops_per_token: float  # 2 x (parameters of the layers' products)
    head_flops_per_row: float  # 2 x vocabulary x hidden
    attention_flops_per_pair: float  # per (query, key) pair, all layers: 4 x heads x head_dim x layers

    def step(self, spans: list[tuple[int, int]], logit_rows: int) -> tuple[float, float]:
        """(bytes, flops) of a step whose requests bring ``spans`` = (cached, new) tokens."""
        new = sum(n for _, n in spans)
        held = sum(c + n for c, n in spans)
        pairs = sum(n * c + n * (n + 1) // 2 for c, n in spans)
        return (self.weight_bytes + held * self.kv_bytes_per_token,
                new * self.linear_flops_per_token + logit_rows * self.head_flops_per_row
                + pairs * self.attention_flops_per_pair)


def step_mix(records: list[StepRecord], cost: ModelCost | None, hbm_gbs: float, tflops: float) -> dict:
    """Steps, tokens and time by kind of step (prefill / decode / mixed) and, with ``cost``, the
    fraction of the roofline each kind reaches: the sum over its steps of max(bytes / bandwidth,
    flops / peak) divided by the time those steps took."""
    out: dict[str, dict] = {}
    for r in records:
        row = out.setdefault(r.kind, dict(steps=0, seconds=0.0, prefill_tokens=0, decode_tokens=0, ideal_s=0.0))
        row["steps"] += 1
        row["seconds"] += r.seconds
        row["prefill_tokens"] += r.prefill_tokens
        row["decode_tokens"] += r.decode_tokens
        if cost is not None and r.spans:
            nbytes, flops = cost.step(r.spans, len(r.spans))
            row["ideal_s"] += max(nbytes / (hbm_gbs * 1e9), flops / (tflops * 1e12))
    for row in out.values():
        row["roofline_frac"] = round(row["ideal_s"] / row["seconds"], 4) if row["ideal_s"] and row["seconds"] else None
        row["ms_per_step"] = round(1e3 * row["seconds"] / row["steps"], 3)
        row["seconds"] = round(row["seconds"], 4)
        del row["ideal_s"]
    out["preemptions"] = sum(r.preempts for r in records)
    return out
