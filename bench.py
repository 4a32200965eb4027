#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, with roofline fractions.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

The default run has the layer sizes of Qwen3-4B (36 layers, hidden 2560, 32/8 heads of
128, feed-forward 9728, vocabulary 151936, tied head) with seeded random bfloat16 weights,
a batch of 8 requests and a context of 4096 tokens per request.  A *step* is one decode
step: every live request gets one new token.  It prints ONE JSON line:

* ``value``     decoded tokens per second, timed on the device with CUDA events around
                exactly K step-function calls (metadata copy, all kernels, logits); three
                such regions are timed and the one with the median time is reported
                (``trials_ms`` lists all three);
* ``e2e``       the same through the public engine API (``Engine.step``): scheduling, the
                pinned host->device copy of the step's inputs, the kernels, sampling and
                the device->host read of the new token ids (the engine runs ahead: a step's
                ids are read while the next step, fed from the device, already runs; every
                step's inputs are still copied in and every step's ids still read out).
                Between the prefill of the prompts and the W warm-up steps both arms decode 40
                untimed steps: right after a prefill at the power cap decode steps run up to
                15 % slower for some 40 ms, which is not what a step costs;
* ``prefill``   one 2,048-token prompt through the step function;
* ``roofline``  bytes a decode step has to read (every weight once + the live requests'
                keys and values) / its time, against the measured copy bandwidth;
* ``points``    decode tokens per second at batch 1 and 64 (same context);
* ``kernels``   per kernel of one eager decode step and one eager prefill step: launches,
                microseconds (CUDA events around each launch), algorithmic bytes or flops and
                the fraction of the measured peak (burst peaks: each kernel is timed alone).

``--workload`` runs another workload instead and prints one line of the same form
(``value`` is then the workload's output tokens per second, end to end through
``build_engine`` / ``add_request`` / ``Engine.step``; one warm-up trial and the median of
``--trials`` timed ones, with time to first token, time per output token, the mix of step
kinds and a roofline fraction per kind):

* ``decode512``    Qwen3-4B sizes, B = 1 / 8 / 64 requests of 512 prompt ids decoding 512 tokens;
* ``batch48``      Qwen3-8B sizes (untied head), 48 requests with prompt lengths uniform in
                   [64, 4096] and 256 output tokens, token budgets 2048 and 8192;
* ``32b``          Qwen3-32B sizes: decode at B = 1 / 8 / 32 behind 1,024-id prompts and one
                   2,048-token prefill (device-timed), and B = 8 end to end;
* ``decode``, ``latency``, ``batch8``, ``throughput``, ``prefill``, ``longctx``: the six closed
                   batches of the reference's own harness (bench/workloads.py:34-43) at Qwen3-4B
                   sizes, with its token budget rule (bench/workloads.py:52-64).

Weights (8 GB and more) are far larger than the 126 MB L2, so no L2 flush is needed between
timed iterations.  ``--impl reference`` runs the unmodified reference installed under
``baseline/_ref`` on the same workload.  More than one GPU is not supported.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# layer sizes of the three models the measurements name (docs/pins/Qwen3-4B/config.json of the
# reference for the first; the published Qwen3-8B and Qwen3-32B config.json for the others)
SHAPES = {
    "4b": dict(vocab_size=151936, hidden_size=2560, num_hidden_layers=36, num_attention_heads=32,
               num_key_value_heads=8, head_dim=128, intermediate_size=9728, rms_norm_eps=1e-6, rope_theta=1e6,
               max_position_embeddings=40960, tie_word_embeddings=True),
    "8b": dict(vocab_size=151936, hidden_size=4096, num_hidden_layers=36, num_attention_heads=32,
               num_key_value_heads=8, head_dim=128, intermediate_size=12288, rms_norm_eps=1e-6, rope_theta=1e6,
               max_position_embeddings=40960, tie_word_embeddings=False),
    "32b": dict(vocab_size=151936, hidden_size=5120, num_hidden_layers=64, num_attention_heads=64,
                num_key_value_heads=8, head_dim=128, intermediate_size=25600, rms_norm_eps=1e-6, rope_theta=1e6,
                max_position_embeddings=40960, tie_word_embeddings=False),
}
SHAPE = SHAPES["4b"]
CONTEXT = 4096
BATCH = 8
PREFILL_TOKENS = 2048
PAGE = 16
SEED = 20260825
# the reference's own closest published number: batch8 output tok/s on an RTX 4090-class GPU
BASELINE_TOK_S = 693.26

# (concurrency = requests, prompt tokens, output tokens) of the reference's closed batches
CLOSED_CASES = {"decode": (1, 256, 512), "latency": (1, 512, 128), "batch8": (8, 256, 128),
                "throughput": (16, 256, 128), "prefill": (1, 2048, 16), "longctx": (1, 8192, 64)}
WORKLOADS = ("default", "decode512", "batch48", "32b", *CLOSED_CASES)


def peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        raw = json.loads(path.read_text())
        burst = float(raw.get("bf16_tflops", 1590.0))
        return dict(hbm_gbs=float(raw.get("hbm_gbs", 6650.0)), bf16_tflops=float(raw.get("bf16_tflops_sustained", burst)),
                    bf16_tflops_burst=burst, source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_burst=1590.0, source="fallback")


E2E_SETTLE_STEPS = 40  # untimed decode steps between the prompts' prefill and the W warm-up steps (e2e_steps)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi.  The process runs from ``start()`` to
    ``close()``; samples are kept only inside ``with sampler:`` (a timed region), so that building a
    model or writing its folder, with the GPU idle, does not enter the record."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.samples: list[list[str]] = []
        self.proc = None
        self.index = index
        self.keeping = 0

    def start(self):
        if self.proc is None:
            try:
                self.proc = subprocess.Popen(
                    ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                     "--format=csv,noheader,nounits", "-lms", "100"],
                    stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
                self.thread = threading.Thread(target=self._read, daemon=True)
                self.thread.start()
            except OSError:
                self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6 and self.keeping:
                self.samples.append(parts)

    def __enter__(self):
        self.start()
        self.keeping += 1
        return self

    def __exit__(self, *exc):
        if self.keeping == 1:
            time.sleep(0.12)  # the sample that covers the end of the region
        self.keeping -= 1

    def close(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.proc = None

    def summary(self) -> dict:
        self.close()
        sm = [int(s[0]) for s in self.samples if s[0].isdigit()]
        mx = [int(s[1]) for s in self.samples if s[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return dict(sm_mhz=int(statistics.median(sm)) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=reasons, samples=len(sm))


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


def flat_config(cfg, *, model: str, batch, seq_len, layers_full: int, cuda_graph=True, run_ahead=True,
                build_s=0.0) -> dict:
    """The ``config`` record: every size of the model, flat, the same keys for both arms."""
    return {
        "model": model, "global_batch": batch, "seq_len": seq_len, "parallelism": "none",
        "layers": cfg.num_hidden_layers, "layers_full": layers_full, "hidden": cfg.hidden_size,
        "q_heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
        "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "tied_head": cfg.tie_word_embeddings,
        "page_size": PAGE, "cuda_graph": bool(cuda_graph), "l2": "inputs (GBs of weights) larger than L2",
        "run_ahead": bool(run_ahead), "build_s": round(build_s, 1), "e2e_steps_after_prefill": E2E_SETTLE_STEPS,
    }


def model_cost(cfg):
    """Bytes and flops of a step from the model's sizes (engine/harness.py: ModelCost)."""
    from qwen3_runtime_b200.engine.harness import ModelCost

    L, H, I, V = cfg.num_hidden_layers, cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    q, kv = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    per_layer = H * (q + 2 * kv) + q * H + 3 * H * I
    return ModelCost(weight_bytes=2.0 * (L * per_layer + V * H), kv_bytes_per_token=2.0 * 2 * kv * L,
                     linear_flops_per_token=2.0 * L * per_layer, head_flops_per_row=2.0 * V * H,
                     attention_flops_per_pair=4.0 * cfg.num_attention_heads * cfg.head_dim * L)


# ------------------------------------------------------------------------------------------
# this engine
# ------------------------------------------------------------------------------------------

def build_ours(shape_name: str, args, *, max_num_seqs: int, budget: int, tokens_needed: int, cuda_graph=True):
    """(engine, model, cfg, ops, seconds to build) for a named shape with random device weights."""
    import torch

    from qwen3_runtime_b200.config import Qwen3Config
    from qwen3_runtime_b200.engine.factory import build_engine, build_model
    from qwen3_runtime_b200.ops.cuda import CudaOps
    from qwen3_runtime_b200.weights.random_init import RandomDeviceSource, expected_tensors_for

    shape = dict(SHAPES[shape_name])
    if args.layers:
        shape["num_hidden_layers"] = args.layers
    cfg = Qwen3Config(**shape)
    torch.cuda.set_device(0)
    ops = CudaOps()
    t0 = time.time()
    model = build_model(cfg, RandomDeviceSource(expected_tensors_for(cfg), SEED, "cuda"), dtype="bfloat16", ops=ops)
    torch.cuda.synchronize()
    build_s = time.time() - t0
    engine = build_engine(model=model, config=cfg, max_num_seqs=max_num_seqs, max_num_batched_tokens=budget,
                          block_size=PAGE, num_kv_blocks=-(-tokens_needed // PAGE), cuda_graph=cuda_graph)
    return engine, model, cfg, ops, build_s


def make_rand_ids(torch):
    gen = torch.Generator().manual_seed(SEED)

    def rand_ids(n):
        return torch.randint(1, 1000, (n,), generator=gen).tolist()

    return rand_ids


def decode_point(rt, ops, torch, rand_ids, batch: int, context: int, steps: int, warmup: int, regions: int = 1,
                 sampler=None):
    """Device-timed decode steps through the step function (``runner.run``): ``regions`` timed
    regions of exactly ``steps`` steps each after ``warmup`` untimed ones; returns the list of
    milliseconds per step (one per region) and the launches per step."""
    from qwen3_runtime_b200.engine.batch import StepEntry

    handles = []
    for i in range(batch):
        rc = rt.cache.open(("bench", batch, i))
        rt.cache.reserve(rc, context)
        rt.cache.commit(rc, context)
        rc.needs_state_reset = False
        handles.append(rc)
    total = warmup + regions * steps
    ids = [rand_ids(total + 1) for _ in range(batch)]

    def one(step_no):
        entries = []
        for rc, toks in zip(handles, ids):
            rt.cache.reserve(rc, 1)
            entries.append(StepEntry(rc, [toks[step_no]], [0]))
        return rt.runner.run(entries)

    for s in range(warmup):
        one(s)
    torch.cuda.synchronize()
    before = ops.launches
    out = []
    with (sampler if sampler is not None else _Null()):
        for r in range(regions):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            for s in range(warmup + r * steps, warmup + (r + 1) * steps):
                one(s)
            stop.record()
            torch.cuda.synchronize()
            out.append(start.elapsed_time(stop) / steps)
    launches = (ops.launches - before) / (regions * steps)
    for rc in handles:
        rt.cache.close(rc)
    return out, launches


def prefill_point(rt, torch, rand_ids, tokens: int, repeats: int = 3) -> float:
    """Median milliseconds of one ``tokens``-token prompt through the step function."""
    from qwen3_runtime_b200.engine.batch import StepEntry

    def once():
        rc = rt.cache.open("prefill")
        rt.cache.reserve(rc, tokens)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        toks = rand_ids(tokens)
        torch.cuda.synchronize()
        start.record()
        rt.runner.run([StepEntry(rc, toks, [tokens - 1])])
        stop.record()
        torch.cuda.synchronize()
        rt.cache.close(rc)
        return start.elapsed_time(stop)

    for _ in range(3):
        once()
    return statistics.median(once() for _ in range(repeats))


def kernel_table(rt, ops, torch, rand_ids, batch: int, context: int, pk: dict) -> list[dict]:
    """One eager decode step and one eager prefill step with CUDA events around every launch of
    the kernel table: per kernel launches, microseconds, bytes or flops and the fraction of the
    measured peak (burst: each kernel runs alone between its events)."""
    from qwen3_runtime_b200.engine.batch import StepEntry

    rows = []
    for kind in ("decode", "prefill"):
        handles = []
        if kind == "decode":
            for i in range(batch):
                rc = rt.cache.open(("kernels", i))
                rt.cache.reserve(rc, context + 2)
                rt.cache.commit(rc, context)
                rc.needs_state_reset = False
                handles.append(rc)
            make = lambda: [StepEntry(rc, rand_ids(1), [0]) for rc in handles]  # noqa: E731
        else:
            rc = rt.cache.open("kernels-prefill")
            rt.cache.reserve(rc, PREFILL_TOKENS)
            handles.append(rc)
            toks = rand_ids(PREFILL_TOKENS)
            make = lambda: [StepEntry(rc, toks, [PREFILL_TOKENS - 1])]  # noqa: E731

        def forward():
            step = rt.runner.builder.build(make(), scratch_page=rt.storage.scratch_page,
                                           scratch_slot=rt.storage.scratch_slot)
            rt.model.forward(step, rt.storage)  # eager, no graph; the cache is not advanced

        forward()  # warm
        torch.cuda.synchronize()
        ops.timing = []
        # keep the device busy while the host enqueues the step, so that every kernel starts the
        # moment its start event is reached and the events time kernels, not launch gaps
        torch.cuda._sleep(150_000_000)
        forward()
        table = ops.timed_kernels()
        ops.timing = None
        for row in table:
            us = row["us"]
            t_mem = row["bytes"] / (pk["hbm_gbs"] * 1e9)
            t_flop = row["flops"] / (pk["bf16_tflops_burst"] * 1e12)
            bound = "flops" if t_flop > t_mem else "hbm"
            rows.append(dict(step=kind, name=row["name"], launches=row["launches"], us=round(us, 1),
                             **({"gflop": round(row["flops"] / 1e9, 2)} if bound == "flops" else
                                {"mbytes": round(row["bytes"] / 1e6, 2)}),
                             bound=bound, frac=round(max(t_mem, t_flop) / (us * 1e-6), 3) if us > 0 else None))
        for rc in handles:
            rt.cache.close(rc)
    return rows


def run_ours(args) -> dict:
    import torch

    K, W = args.steps, args.warmup
    clocks = ClockSampler().start()
    max_b = max(BATCH, 64)
    tokens_needed = max_b * (args.context + 3 * K + W + E2E_SETTLE_STEPS + 64) + PREFILL_TOKENS + 64
    engine, model, cfg, ops, build_s = build_ours("4b", args, max_num_seqs=max_b, budget=8192,
                                                  tokens_needed=tokens_needed)
    rt = engine.runtime
    cost = model_cost(cfg)
    rand_ids = make_rand_ids(torch)
    # the pages of the decode points are filled with random keys and values instead of being
    # computed by a prefill: what a decode step reads and computes does not depend on them
    for t in rt.storage.tensors:
        t.normal_(0.0, 0.5)

    trials, _ = decode_point(rt, ops, torch, rand_ids, BATCH, args.context, K, W, regions=3, sampler=clocks)
    ms_step = statistics.median(trials)
    value = BATCH * 1000.0 / ms_step
    points = {}
    for b in (1, 64):
        ms_b, _ = decode_point(rt, ops, torch, rand_ids, b, args.context, max(8, K // 2), W)
        points[f"decode_b{b}"] = round(b * 1000.0 / ms_b[0], 1)

    # a captured decode step replays the kernels of one eager forward: count those
    per_forward = _launches_of_one_forward(rt, ops, BATCH, args.context, rand_ids)
    gpu_launches = int(per_forward * K)

    pk = peaks()
    prefill_ms = prefill_point(rt, torch, rand_ids, PREFILL_TOKENS)
    _bytes, prefill_flops = cost.step([(0, PREFILL_TOKENS)], 1)
    prefill = dict(value=round(PREFILL_TOKENS * 1000.0 / prefill_ms, 1), tokens=PREFILL_TOKENS,
                   ms=round(prefill_ms, 3),
                   frac=round(prefill_flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4))

    # roofline of the decode step: the region with the median time started after W + r*K steps
    region = trials.index(ms_step)
    held = args.context + W + region * K + K / 2
    step_bytes = cost.weight_bytes + BATCH * held * cost.kv_bytes_per_token
    achieved = step_bytes / (ms_step * 1e-3) / 1e9
    roofline = dict(bound="hbm", achieved=round(achieved, 1), peak=pk["hbm_gbs"], unit="GB/s",
                    frac=round(achieved / pk["hbm_gbs"], 4), peak_source=pk["source"])

    kernels = kernel_table(rt, ops, torch, rand_ids, BATCH, args.context, pk)
    e2e = e2e_ours(engine, args, rand_ids, torch)

    return {
        "metric": "decode tok/s @ batch 8, ctx 4096 (Qwen3-4B shape, bf16)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": round(value / BASELINE_TOK_S, 3), "dtype": "bf16",
        "data": "synthetic: seeded random weights N(0,0.02), random token ids; pages of the decode points hold random keys/values",
        "impl": "ours",
        "config": flat_config(cfg, model="Qwen3-4B shape", batch=BATCH, seq_len=args.context,
                              layers_full=SHAPE["num_hidden_layers"], run_ahead=engine.config.run_ahead,
                              build_s=build_s),
        "e2e": e2e, "prefill": prefill, "roofline": roofline, "points": points,
        "trials_ms": [round(t, 4) for t in trials],
        "gpu_launches": gpu_launches, "clocks": clocks.summary(), "kernels": kernels,
    }


def _launches_of_one_forward(rt, ops, batch, context, rand_ids) -> int:
    """Kernels of this engine launched by one decode forward (eager, outside a graph)."""
    import torch

    from qwen3_runtime_b200.engine.batch import StepEntry

    handles = []
    for i in range(batch):
        rc = rt.cache.open(("count", i))
        rt.cache.reserve(rc, context + 1)
        rt.cache.commit(rc, context)
        rc.needs_state_reset = False
        handles.append(rc)
    entries = [StepEntry(rc, rand_ids(1), [0]) for rc in handles]
    step = rt.runner.builder.build(entries, scratch_page=rt.storage.scratch_page, scratch_slot=rt.storage.scratch_slot)
    before = ops.launches
    rt.model.forward(step, rt.storage)
    torch.cuda.synchronize()
    count = ops.launches - before
    for rc in handles:
        rt.cache.close(rc)
    return count


def e2e_steps(engine, torch, batch: int, context: int, K: int, W: int, rand_ids, make_sampling) -> dict:
    """Decode steps through ``engine.step()``: host token ids in, sampled ids out, every step.
    Works for this engine and for the reference's (the same three calls)."""
    prompts = [rand_ids(context) for _ in range(batch)]
    rids = [engine.add_request(p, max_tokens=E2E_SETTLE_STEPS + W + K + 8, sampling=make_sampling())
            for p in prompts]
    produced = {rid: 0 for rid in rids}

    def step():
        n = 0
        for rid, tok, _fin in engine.step():
            if tok is not None:
                produced[rid] = produced.get(rid, 0) + 1
                n += 1
        return n

    while any(produced[r] < 1 for r in rids):
        step()  # untimed: the prompts are prefilled in portions of the token budget
    # the prefill of batch x context tokens runs at the power cap; the decode steps right after it
    # are up to 15 % slower for some 40 ms while the clocks come back (and an idle pause instead
    # lets them fall).  Both arms decode E2E_SETTLE_STEPS untimed steps first, so that the timed
    # steps are steady-state decode steps.
    for _ in range(E2E_SETTLE_STEPS + W):
        step()
    ahead_before = getattr(engine, "num_run_ahead", 0)
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    t0 = time.perf_counter()
    tokens = sum(step() for _ in range(K))
    stop.record()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    device_ms = start.elapsed_time(stop)
    for rid in rids:
        if hasattr(engine, "abort_request"):
            engine.abort_request(rid)
    return dict(tokens=tokens, seconds=dt, device_ms=device_ms,
                steps_run_ahead=getattr(engine, "num_run_ahead", 0) - ahead_before)


def e2e_ours(engine, args, rand_ids, torch, batch: int = BATCH, context: int | None = None) -> dict:
    from qwen3_runtime_b200.sampling.params import SamplingParams

    K, W = args.steps, args.warmup
    context = context or args.context
    r = e2e_steps(engine, torch, batch, context, K, W, rand_ids, SamplingParams)
    # per step: ids, positions, sequence index, logit rows (4 B each per request), cu_seqlens,
    # kv_lens, slots, and one block-table row per request; back: one int32 token id per request
    width = 1 << ((context + E2E_SETTLE_STEPS + W + K + 8) // PAGE).bit_length()
    h2d = 4 * (4 * batch + (batch + 1) + 2 * batch + batch * width)
    return dict(value=round(r["tokens"] / r["seconds"], 1), unit="tokens/s",
                ms_per_step=round(r["seconds"] * 1000.0 / K, 4), h2d_bytes_per_step=h2d,
                d2h_bytes_per_step=4 * batch, steps=K, steps_run_ahead=r["steps_run_ahead"])


# ------------------------------------------------------------------------------------------
# workloads run end to end under the scheduler (both arms)
# ------------------------------------------------------------------------------------------

def closed_batch_trials(engine, prompts, max_tokens, trials: int, cost, pk, torch, clocks=None) -> dict:
    """One warm-up run and ``trials`` timed runs of a closed batch; medians over the trials, the
    step mix of the last one."""
    from qwen3_runtime_b200.engine.harness import run_closed_batch, step_mix, summarize

    runs = []
    for i in range(1 + trials):
        ahead = getattr(engine, "num_run_ahead", 0)
        with (clocks if clocks is not None and i > 0 else _Null()):
            traces, records, wall = run_closed_batch(engine, prompts, max_tokens, synchronize=torch.cuda.synchronize)
        if i == 0:
            continue  # warm-up: kernels loaded, graphs captured
        s = summarize(traces, wall)
        s["steps_run_ahead"] = getattr(engine, "num_run_ahead", 0) - ahead
        s["mix"] = step_mix(records, cost, pk["hbm_gbs"], pk["bf16_tflops"])
        runs.append(s)
    med = lambda xs: statistics.median(xs) if xs else None  # noqa: E731
    last = runs[-1]
    return dict(
        output_tok_s=round(med([r["output_tok_s"] for r in runs]), 1),
        output_tok_s_trials=[round(r["output_tok_s"], 1) for r in runs],
        ttft_ms=_ms(med([r["ttft_s"]["median"] for r in runs if r["ttft_s"]["median"] is not None])),
        tpot_ms=_ms(med([r["tpot_s"]["median"] for r in runs if r["tpot_s"]["median"] is not None])),
        wall_s=round(med([r["wall_s"] for r in runs]), 3), forced_length_ok=all(r["forced_length_ok"] for r in runs),
        requests=last["n_requests"], output_tokens=last["output_tokens"], steps_run_ahead=last["steps_run_ahead"],
        step_mix=last["mix"], trials=len(runs))


def _ms(x):
    return None if x is None else round(1e3 * x, 3)


def workload_prompts(name: str, np):
    """Prompts (uniform ids in [1, 1000), the reference's rule, bench/workloads.py:82-86), output
    lengths and engine sizes of a named workload: ``[(label, shape, prompts, max_tokens, max_num_seqs,
    token budget)]``."""
    rng = np.random.default_rng(SEED)
    out = []
    if name in CLOSED_CASES:
        n, p, o = CLOSED_CASES[name]
        budget = 2048 if name == "longctx" else max(2048, n * p)  # bench/workloads.py:52-64
        out.append((name, "4b", rng.integers(1, 1000, size=(n, p)).tolist(), o, n, budget))
    elif name == "decode512":
        for b in (1, 8, 64):
            out.append((f"b{b}", "4b", rng.integers(1, 1000, size=(b, 512)).tolist(), 512, b, max(2048, b * 512)))
    elif name == "batch48":
        lens = rng.integers(64, 4097, size=48)
        prompts = [rng.integers(1, 1000, size=int(n)).tolist() for n in lens]
        for budget in (2048, 8192):
            out.append((f"budget{budget}", "8b", prompts, 256, 48, budget))
    return out


def run_workload_ours(args) -> dict:
    import numpy as np
    import torch

    pk = peaks()
    if args.workload == "32b":
        return run_32b_ours(args, pk)
    cases = workload_prompts(args.workload, np)
    results, cfg, build_s, engine = {}, None, 0.0, None
    clocks = ClockSampler()
    clocks.start()
    for label, shape, prompts, max_tokens, seqs, budget in cases:
        tokens = sum(len(p) for p in prompts) + len(prompts) * (max_tokens + 2 * PAGE)
        engine, model, cfg, ops, build_s = build_ours(shape, args, max_num_seqs=seqs, budget=budget,
                                                      tokens_needed=tokens + 64)
        results[label] = closed_batch_trials(engine, prompts, max_tokens, args.trials, model_cost(cfg), pk, torch,
                                             clocks=clocks)
        results[label]["max_num_batched_tokens"] = budget
        ops.raise_if_kernel_error()
        del engine, model
        torch.cuda.empty_cache()
    first = next(iter(results.values()))
    shape = cases[0][1]
    return _workload_line(args, "ours", shape, cfg, results, first, clocks, build_s, pk)


def _workload_line(args, impl, shape, cfg, results, headline, clocks, build_s, pk, extra=None) -> dict:
    names = {"4b": "Qwen3-4B shape", "8b": "Qwen3-8B shape", "32b": "Qwen3-32B shape"}
    line = {
        "metric": f"output tok/s, workload {args.workload} ({names[shape]}, bf16, end to end under the scheduler)",
        "value": headline["output_tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": headline.get("output_tokens"),
        "warmup": 1, "ms_per_step": headline.get("tpot_ms"), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "impl": impl, "workload": args.workload,
        "data": "synthetic: seeded random weights N(0,0.02), uniform random token ids in [1, 1000)",
        "config": flat_config(cfg, model=names[shape], batch=headline.get("requests"), seq_len="per workload",
                              layers_full=SHAPES[shape]["num_hidden_layers"], build_s=build_s),
        "results": results, "peaks": pk, "clocks": clocks.summary(),
    }
    if extra:
        line.update(extra)
    return line


def run_32b_ours(args, pk) -> dict:
    """Qwen3-32B sizes on one B200: device-timed decode at B = 1 / 8 / 32 behind 1,024-token
    contexts, one 2,048-token prefill, and B = 8 end to end through the engine."""
    import torch

    K, W = args.steps, args.warmup
    context = 1024
    tokens = (32 * (context + 2 * K + W + 64) + 8 * (context + K + W + E2E_SETTLE_STEPS + 64)
              + PREFILL_TOKENS + 64)
    engine, model, cfg, ops, build_s = build_ours("32b", args, max_num_seqs=32, budget=8192, tokens_needed=tokens)
    rt = engine.runtime
    cost = model_cost(cfg)
    rand_ids = make_rand_ids(torch)
    for t in rt.storage.tensors:
        t.normal_(0.0, 0.5)
    clocks = ClockSampler()
    results = {}
    clocks.start()
    for b in (1, 8, 32):
        trials, _ = decode_point(rt, ops, torch, rand_ids, b, context, K, W, regions=3, sampler=clocks)
        ms = statistics.median(trials)
        nbytes = cost.weight_bytes + b * (context + W + 1.5 * K) * cost.kv_bytes_per_token
        results[f"decode_b{b}"] = dict(tok_s=round(b * 1e3 / ms, 1), ms_per_step=round(ms, 4),
                                       trials_ms=[round(t, 4) for t in trials],
                                       hbm_frac=round(nbytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4))
    prefill_ms = prefill_point(rt, torch, rand_ids, PREFILL_TOKENS)
    _b, flops = cost.step([(0, PREFILL_TOKENS)], 1)
    results["prefill_2048"] = dict(tok_s=round(PREFILL_TOKENS * 1e3 / prefill_ms, 1), ms=round(prefill_ms, 3),
                                   frac=round(flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4))
    e2e = e2e_ours(engine, args, rand_ids, torch, batch=8, context=context)
    ops.raise_if_kernel_error()
    head = dict(output_tok_s=results["decode_b8"]["tok_s"], tpot_ms=results["decode_b8"]["ms_per_step"], requests=8,
                output_tokens=K)
    free, total = torch.cuda.mem_get_info()
    return _workload_line(args, "ours", "32b", cfg, results, head, clocks, build_s, pk,
                          extra={"e2e": e2e, "device_memory_gb": dict(used=round((total - free) / 1e9, 1),
                                                                     total=round(total / 1e9, 1))})


# ------------------------------------------------------------------------------------------
# the reference, unmodified, from baseline/_ref
# ------------------------------------------------------------------------------------------

def _reference_engine(args, shape_name: str, *, max_num_seqs: int, budget: int, tokens_needed: int):
    """The reference's own ``build_engine`` on a random model folder of the named shape."""
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "qwen3_runtime").is_dir():
        raise RuntimeError("baseline/_ref is not installed (pip --target baseline/_ref)")
    if str(ref) not in sys.path:
        sys.path.insert(0, str(ref))
    import torch

    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device")
    from qwen3_runtime.engine.factory import build_engine as ref_build_engine  # the reference's public API

    from qwen3_runtime_b200.config import Qwen3Config
    from qwen3_runtime_b200.weights.random_init import write_random_model

    shape = dict(SHAPES[shape_name])
    if args.layers:
        shape["num_hidden_layers"] = args.layers
    cfg = Qwen3Config(**shape)
    folder = Path(tempfile.mkdtemp(prefix="q3ref_"))
    t0 = time.time()
    write_random_model(cfg, folder, SEED)  # same distributions as our arm; values differ (CPU generator)
    write_s = time.time() - t0
    kv_budget = tokens_needed * 2 * cfg.num_hidden_layers * cfg.num_key_value_heads * cfg.head_dim * 2
    engine = ref_build_engine(str(folder), max_num_seqs=max_num_seqs, max_num_batched_tokens=budget,
                              block_size=PAGE, pin=False, kv_budget=kv_budget)
    return engine, cfg, write_s, folder


def run_reference(args) -> dict:
    try:
        import torch

        K, W = args.steps, args.warmup
        engine, cfg, write_s, _folder = _reference_engine(args, "4b", max_num_seqs=BATCH, budget=8192,
                                                          tokens_needed=BATCH * (args.context + K + W
                                                                                 + E2E_SETTLE_STEPS + 64))
        from qwen3_runtime.sampling_params import SamplingParams as RefSamplingParams

        clocks = ClockSampler()
        with clocks:
            r = e2e_steps(engine, torch, BATCH, args.context, K, W, make_rand_ids(torch), RefSamplingParams)
        ms = r["device_ms"] / K
        value = r["tokens"] / (r["device_ms"] * 1e-3)
        return {
            "metric": "decode tok/s @ batch 8, ctx 4096 (Qwen3-4B shape, bf16)", "impl": "reference",
            "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
            "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": round(value / BASELINE_TOK_S, 3), "dtype": "bf16",
            "data": "synthetic: seeded random weights N(0,0.02), random token ids",
            "config": flat_config(cfg, model="Qwen3-4B shape", batch=BATCH, seq_len=args.context,
                                  layers_full=SHAPE["num_hidden_layers"], cuda_graph=engine.config.cuda_graph,
                                  run_ahead=False, build_s=write_s),
            "reference_info": {"attention_backend": engine.config.attention_backend, "write_model_s": round(write_s, 1)},
            "e2e": dict(value=round(r["tokens"] / r["seconds"], 1), unit="tokens/s",
                        ms_per_step=round(r["seconds"] * 1000.0 / K, 4)),
            "clocks": clocks.summary(),
        }
    except Exception as exc:  # noqa: BLE001 - the arm reports why it could not run
        return {"impl": "reference", "unavailable": f"{type(exc).__name__}: {str(exc).splitlines()[0][:200]}"}


def run_workload_reference(args) -> dict:
    """The reference's engine on a named workload, through the same closed-batch loop."""
    if args.workload == "32b":
        return {"impl": "reference", "workload": "32b",
                "unavailable": "the reference loads weights from safetensors files only; a random Qwen3-32B-shaped "
                               "checkpoint is 65 GB to draw on the CPU and write to disk before its loader reads it "
                               "back, beyond what a benchmark run can spend"}
    try:
        import numpy as np
        import torch

        pk = peaks()
        cases = workload_prompts(args.workload, np)
        results, cfg, write_s = {}, None, 0.0
        clocks = ClockSampler()
        clocks.start()
        for label, shape, prompts, max_tokens, seqs, budget in cases:
            tokens = sum(len(p) for p in prompts) + len(prompts) * (max_tokens + 2 * PAGE) + 64
            engine, cfg, write_s, folder = _reference_engine(args, shape, max_num_seqs=seqs, budget=budget,
                                                             tokens_needed=tokens)
            results[label] = closed_batch_trials(engine, prompts, max_tokens, args.trials, None, pk, torch,
                                                 clocks=clocks)
            results[label]["max_num_batched_tokens"] = budget
            results[label]["attention_backend"] = engine.config.attention_backend
            del engine
            torch.cuda.empty_cache()
            for f in folder.iterdir():
                f.unlink()
            folder.rmdir()
        first = next(iter(results.values()))
        return _workload_line(args, "reference", cases[0][1], cfg, results, first, clocks, write_s, pk)
    except Exception as exc:  # noqa: BLE001 - the arm reports why it could not run
        return {"impl": "reference", "workload": args.workload,
                "unavailable": f"{type(exc).__name__}: {str(exc).splitlines()[0][:200]}"}


def run_profile_step(args) -> dict:
    """A few eager (not graph-replayed) steps of one kind, for a profiler to list kernels:
    ``--only decode`` (``--batch`` requests of ``--context`` tokens), ``--only prefill``, or
    ``--only mixed`` (a 512-token portion beside ``--batch`` decoding requests)."""
    import torch

    from qwen3_runtime_b200.config import Qwen3Config
    from qwen3_runtime_b200.engine.batch import StepEntry
    from qwen3_runtime_b200.engine.factory import build_model, build_runtime
    from qwen3_runtime_b200.ops.cuda import CudaOps
    from qwen3_runtime_b200.weights.random_init import RandomDeviceSource, expected_tensors_for

    shape = dict(SHAPES[args.shape])
    if args.layers:
        shape["num_hidden_layers"] = args.layers
    cfg = Qwen3Config(**shape)
    ops = CudaOps()
    model = build_model(cfg, RandomDeviceSource(expected_tensors_for(cfg), SEED, "cuda"), dtype="bfloat16", ops=ops)
    tokens = args.batch * (args.context + args.steps + args.warmup + 64) + (args.steps + args.warmup + 1) * PREFILL_TOKENS
    rt = build_runtime(model, block_size=PAGE, num_kv_blocks=-(-tokens // PAGE), max_num_seqs=args.batch + 1,
                       cuda_graph=args.graph)
    gen = torch.Generator().manual_seed(SEED)
    times = []
    handles = []
    if args.only in ("decode", "mixed"):
        for i in range(args.batch):
            rc = rt.cache.open(i)
            rt.cache.reserve(rc, args.context)
            rt.cache.commit(rc, args.context)
            handles.append(rc)
    for s in range(args.warmup + args.steps):
        entries = []
        for rc in handles:
            rt.cache.reserve(rc, 1)
            entries.append(StepEntry(rc, torch.randint(1, 1000, (1,), generator=gen).tolist(), [0]))
        portion = None
        if args.only in ("prefill", "mixed"):
            n = PREFILL_TOKENS if args.only == "prefill" else 512
            portion = rt.cache.open("p")
            rt.cache.reserve(portion, n)
            entries.append(StepEntry(portion, torch.randint(1, 1000, (n,), generator=gen).tolist(), [n - 1]))
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        rt.runner.run(entries)
        torch.cuda.synchronize()
        times.append((time.perf_counter() - t0) * 1e3)
        if portion is not None:
            rt.cache.close(portion)
    return {"only": args.only, "shape": args.shape, "batch": args.batch, "context": args.context,
            "layers": cfg.num_hidden_layers, "graph": args.graph,
            "ms_per_step_wall": [round(t, 3) for t in times[args.warmup:]]}


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--workload", default="default", choices=WORKLOADS)
    parser.add_argument("--trials", type=int, default=3, help="timed runs of a --workload (after one warm-up run)")
    parser.add_argument("--layers", type=int, default=0, help="fewer layers than the full model (0 = all)")
    parser.add_argument("--context", type=int, default=CONTEXT)
    parser.add_argument("--only", choices=["decode", "prefill", "mixed"], default=None,
                        help="run just a few steps of one kind (for profilers); prints wall times")
    parser.add_argument("--shape", choices=sorted(SHAPES), default="4b", help="layer sizes of the --only steps")
    parser.add_argument("--batch", type=int, default=BATCH, help="batch of the --only decode steps")
    parser.add_argument("--graph", action=argparse.BooleanOptionalAction, default=False,
                        help="--only: replay decode steps from a CUDA graph")
    args = parser.parse_args()
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) > 1:
        print("bench.py: this engine runs on ONE GPU; --gpus > 1 is not supported")
        return 2
    if args.only:
        print(json.dumps(run_profile_step(args)))
        return 0
    args.warmup = max(3, args.warmup)
    if args.workload == "default":
        result = run_reference(args) if args.impl == "reference" else run_ours(args)
    else:
        result = run_workload_reference(args) if args.impl == "reference" else run_workload_ours(args)
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
