#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, with roofline fractions.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

The default run has the layer sizes of Qwen3-4B (36 layers, hidden 2560, 32/8 heads of
128, feed-forward 9728, vocabulary 151936, tied head) with seeded random bfloat16 weights,
a batch of 8 requests and a context of 4096 tokens per request.  A *step* is one decode
step: every live request gets one new token.  It prints ONE JSON line:

* ``value``     decoded tokens per second, timed on the device with CUDA events around
                exactly K step-function calls (metadata copy, all kernels, logits);
* ``e2e``       the same through the public engine API (``Engine.step``): scheduling, the
                pinned host->device copy of the step's inputs, the kernels, sampling and
                the device->host read of the new token ids (the engine runs ahead: a step's
                ids are read while the next step, fed from the device, already runs; every
                step's inputs are still copied in and every step's ids still read out);
* ``prefill``   one 2,048-token prompt through the step function;
* ``roofline``  bytes a decode step has to read (every weight once + the live requests'
                keys and values) / its time, against the measured copy bandwidth;
* ``points``    decode tokens per second at batch 1 and 64 (same context).

Weights (8 GB) are far larger than the 126 MB L2, so no L2 flush is needed between
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

# Qwen3-4B layer sizes (docs/pins/Qwen3-4B/config.json of the reference)
SHAPE = dict(vocab_size=151936, hidden_size=2560, num_hidden_layers=36, num_attention_heads=32,
             num_key_value_heads=8, head_dim=128, intermediate_size=9728, rms_norm_eps=1e-6, rope_theta=1e6,
             max_position_embeddings=40960, tie_word_embeddings=True)
CONTEXT = 4096
BATCH = 8
PREFILL_TOKENS = 2048
PAGE = 16
SEED = 20260825
# the reference's own closest published number: batch8 output tok/s on an RTX 4090-class GPU
BASELINE_TOK_S = 693.26


def peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        raw = json.loads(path.read_text())
        return dict(hbm_gbs=float(raw.get("hbm_gbs", 6650.0)),
                    bf16_tflops=float(raw.get("bf16_tflops_sustained", raw.get("bf16_tflops", 1590.0))),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.samples: list[list[str]] = []
        self.proc = None
        self.index = index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.samples.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        sm = [int(s[0]) for s in self.samples if s[0].isdigit()]
        mx = [int(s[1]) for s in self.samples if s[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return dict(sm_mhz=int(statistics.median(sm)) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=reasons, samples=len(sm))


# ------------------------------------------------------------------------------------------
# this engine
# ------------------------------------------------------------------------------------------

def run_ours(args) -> dict:
    import torch

    from qwen3_runtime_b200.config import Qwen3Config
    from qwen3_runtime_b200.engine.batch import StepEntry
    from qwen3_runtime_b200.engine.factory import build_engine, build_model
    from qwen3_runtime_b200.ops.cuda import CudaOps
    from qwen3_runtime_b200.sampling.params import SamplingParams
    from qwen3_runtime_b200.weights.random_init import RandomDeviceSource, expected_tensors_for

    shape = dict(SHAPE)
    layers_full = shape["num_hidden_layers"]
    if args.layers:
        shape["num_hidden_layers"] = args.layers
    cfg = Qwen3Config(**shape)
    torch.cuda.set_device(0)
    ops = CudaOps()
    t0 = time.time()
    source = RandomDeviceSource(expected_tensors_for(cfg), SEED, "cuda")
    model = build_model(cfg, source, dtype="bfloat16", ops=ops)
    torch.cuda.synchronize()
    build_s = time.time() - t0
    K, W = args.steps, args.warmup
    max_b = max(BATCH, 64)
    tokens_needed = max_b * (args.context + K + W + 64) + PREFILL_TOKENS + 64
    engine = build_engine(model=model, config=cfg, max_num_seqs=max_b, max_num_batched_tokens=8192,
                          block_size=PAGE, num_kv_blocks=-(-tokens_needed // PAGE), cuda_graph=True)
    rt = engine.runtime
    layout = model.cache_layout()
    token_bytes = layout.token_bytes(2)
    weight_bytes = sum(
        t.numel() * t.element_size()
        for name, t in _model_tensors(model).items())
    gen = torch.Generator().manual_seed(SEED)

    def rand_ids(n):
        return torch.randint(1, 1000, (n,), generator=gen).tolist()

    # the pages of the decode points are filled with random keys and values instead of being
    # computed by a prefill: what a decode step reads and computes does not depend on them
    for t in rt.storage.tensors:
        t.normal_(0.0, 0.5)

    launches_per_step = {}

    def decode_point(batch: int, steps: int, warmup: int, sampler=None):
        """Device-timed decode steps through the step function (runner.run)."""
        handles = []
        for i in range(batch):
            rc = rt.cache.open(("bench", batch, i))
            rt.cache.reserve(rc, args.context)
            rt.cache.commit(rc, args.context)
            rc.needs_state_reset = False
            handles.append(rc)
        ids = [rand_ids(steps + warmup + 1) for _ in range(batch)]

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
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ctx_mgr = sampler if sampler is not None else _Null()
        with ctx_mgr:
            torch.cuda.synchronize()
            start.record()
            for s in range(warmup, warmup + steps):
                one(s)
            stop.record()
            torch.cuda.synchronize()
        ms = start.elapsed_time(stop) / steps
        launches_per_step[batch] = (ops.launches - before) / steps
        for rc in handles:
            rt.cache.close(rc)
        return ms

    clocks = ClockSampler()
    ms_step = decode_point(BATCH, K, W, clocks)
    value = BATCH * 1000.0 / ms_step
    points = {}
    for b in (1, 64):
        ms_b = decode_point(b, max(8, K // 2), W)
        points[f"decode_b{b}"] = round(b * 1000.0 / ms_b, 1)

    # a captured decode step replays the kernels of one eager forward: count those
    per_forward = _launches_of_one_forward(rt, ops, BATCH, args.context, rand_ids)
    gpu_launches = int(per_forward * K)

    # ---- prefill: one 2,048-token prompt through the step function --------------------------
    def prefill_once():
        rc = rt.cache.open("prefill")
        rt.cache.reserve(rc, PREFILL_TOKENS)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        toks = rand_ids(PREFILL_TOKENS)
        torch.cuda.synchronize()
        start.record()
        rt.runner.run([StepEntry(rc, toks, [PREFILL_TOKENS - 1])])
        stop.record()
        torch.cuda.synchronize()
        rt.cache.close(rc)
        return start.elapsed_time(stop)

    for _ in range(3):
        prefill_once()
    prefill_ms = statistics.median(prefill_once() for _ in range(3))
    L, H, I, V = cfg.num_hidden_layers, cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    q, kv, D = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim, cfg.head_dim
    T = PREFILL_TOKENS
    linear_flops = 2 * T * L * (H * (q + 2 * kv) + q * H + 3 * H * I)
    attn_flops = L * 4 * cfg.num_attention_heads * D * (T * (T + 1) // 2)
    head_flops = 2 * V * H
    prefill_flops = linear_flops + attn_flops + head_flops
    pk = peaks()
    prefill = dict(value=round(T * 1000.0 / prefill_ms, 1), tokens=T, ms=round(prefill_ms, 3),
                   frac=round(prefill_flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4))

    # ---- roofline of the decode step ---------------------------------------------------------
    step_bytes = weight_bytes + BATCH * (args.context + W + K / 2) * token_bytes
    achieved = step_bytes / (ms_step * 1e-3) / 1e9
    roofline = dict(bound="hbm", achieved=round(achieved, 1), peak=pk["hbm_gbs"], unit="GB/s",
                    frac=round(achieved / pk["hbm_gbs"], 4), peak_source=pk["source"])

    # ---- end to end through the public API -----------------------------------------------------
    e2e = e2e_ours(engine, args, rand_ids, torch)

    return {
        "metric": "decode tok/s @ batch 8, ctx 4096 (Qwen3-4B shape, bf16)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": round(value / BASELINE_TOK_S, 3), "dtype": "bf16",
        "data": "synthetic: seeded random weights N(0,0.02), random token ids; pages of the decode points hold random keys/values",
        "impl": "ours",
        "config": {
            "model": "Qwen3-4B shape", "global_batch": BATCH, "seq_len": args.context, "parallelism": "none",
            "layers": cfg.num_hidden_layers, "layers_full": layers_full, "hidden": H, "q_heads": cfg.num_attention_heads,
            "kv_heads": cfg.num_key_value_heads, "head_dim": D, "intermediate": I, "vocab": V,
            "tied_head": cfg.tie_word_embeddings, "page_size": PAGE, "cuda_graph": True,
            "l2": "inputs (8 GB of weights) larger than L2", "run_ahead": bool(engine.config.run_ahead),
            "build_s": round(build_s, 1),
        },
        "e2e": e2e, "prefill": prefill, "roofline": roofline, "points": points,
        "gpu_launches": gpu_launches, "clocks": clocks.summary(),
    }


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


def _model_tensors(model) -> dict:
    """Every weight a decode step reads once (the tied head is the embedding table)."""
    out = {"head": model.head}
    for i, blk in enumerate(model.blocks):
        out[f"{i}.qkv"] = blk.mixer.qkv_weight
        out[f"{i}.o"] = blk.mixer.o_weight
        out[f"{i}.gate_up"] = blk.feed_forward.gate_up_weight
        out[f"{i}.down"] = blk.feed_forward.down_weight
    return out


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


def e2e_ours(engine, args, rand_ids, torch) -> dict:
    """Decode steps through Engine.step(): host token ids in, sampled ids out, every step."""
    from qwen3_runtime_b200.sampling.params import SamplingParams

    K, W = args.steps, args.warmup
    prompts = [rand_ids(args.context) for _ in range(BATCH)]
    reqs = [engine.get_request(engine.add_request(p, max_tokens=W + K + 8, sampling=SamplingParams()))
            for p in prompts]
    while any(not r.is_prefill_complete or r.num_output_tokens < 1 for r in reqs):
        engine.step()  # untimed: the prompts are prefilled in portions of the token budget
    for _ in range(W):
        engine.step()
    torch.cuda.synchronize()
    ahead_before = engine.num_run_ahead
    t0 = time.perf_counter()
    produced = 0
    for _ in range(K):
        produced += sum(1 for _rid, tok, _fin in engine.step() if tok is not None)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    for r in reqs:
        engine.abort_request(r.request_id)
    # per step: ids, positions, sequence index, logit rows (4 B each per request), cu_seqlens,
    # kv_lens, slots, and one block-table row per request; back: one int32 token id per request
    width = 1 << ((args.context + W + K + 8) // PAGE).bit_length()
    h2d = 4 * (4 * BATCH + (BATCH + 1) + 2 * BATCH + BATCH * width)
    return dict(value=round(produced / dt, 1), unit="tokens/s", ms_per_step=round(dt * 1000.0 / K, 4),
                h2d_bytes_per_step=h2d, d2h_bytes_per_step=4 * BATCH, steps=K,
                steps_run_ahead=engine.num_run_ahead - ahead_before)


# ------------------------------------------------------------------------------------------
# the reference, unmodified, from baseline/_ref
# ------------------------------------------------------------------------------------------

def run_reference(args) -> dict:
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "qwen3_runtime").is_dir():
        return {"impl": "reference", "unavailable": "baseline/_ref is not installed (pip --target baseline/_ref)"}
    sys.path.insert(0, str(ref))
    try:
        import torch

        if not torch.cuda.is_available():
            return {"impl": "reference", "unavailable": "no CUDA device"}
        from qwen3_runtime.engine.factory import build_engine as ref_build_engine  # the reference's public API
        from qwen3_runtime.sampling_params import SamplingParams as RefSamplingParams

        from qwen3_runtime_b200.config import Qwen3Config
        from qwen3_runtime_b200.weights.random_init import write_random_model

        shape = dict(SHAPE)
        if args.layers:
            shape["num_hidden_layers"] = args.layers
        cfg = Qwen3Config(**shape)
        K, W = args.steps, args.warmup
        folder = Path(tempfile.mkdtemp(prefix="q3ref_"))
        t0 = time.time()
        write_random_model(cfg, folder, SEED)  # same distributions as our arm; values differ (CPU generator)
        write_s = time.time() - t0
        tokens_needed = BATCH * (args.context + K + W + 64)
        kv_budget = tokens_needed * 2 * cfg.num_hidden_layers * cfg.num_key_value_heads * cfg.head_dim * 2
        engine = ref_build_engine(str(folder), max_num_seqs=BATCH, max_num_batched_tokens=8192, block_size=PAGE,
                                  pin=False, kv_budget=kv_budget)
        gen = torch.Generator().manual_seed(SEED)
        prompts = [torch.randint(1, 1000, (args.context,), generator=gen).tolist() for _ in range(BATCH)]
        rids = [engine.add_request(p, max_tokens=W + K + 8, sampling=RefSamplingParams()) for p in prompts]
        reqs = [engine._requests[r] for r in rids]
        while any(len(r.token_ids) - r.num_prompt_tokens < 1 for r in reqs):
            engine.step()
        for _ in range(W):
            engine.step()
        clocks = ClockSampler()
        with clocks:
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            t0 = time.perf_counter()
            produced = 0
            for _ in range(K):
                produced += sum(1 for _rid, tok, _fin in engine.step() if tok is not None)
            stop.record()
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
        ms = start.elapsed_time(stop) / K
        value = produced / (start.elapsed_time(stop) * 1e-3)
        return {
            "metric": "decode tok/s @ batch 8, ctx 4096 (Qwen3-4B shape, bf16)", "impl": "reference",
            "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
            "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": round(value / BASELINE_TOK_S, 3), "dtype": "bf16",
            "data": "synthetic: seeded random weights N(0,0.02), random token ids",
            "config": {"model": "Qwen3-4B shape", "global_batch": BATCH, "seq_len": args.context, "parallelism": "none",
                       "layers": cfg.num_hidden_layers, "layers_full": SHAPE["num_hidden_layers"],
                       "attention_backend": engine.config.attention_backend, "cuda_graph": engine.config.cuda_graph,
                       "page_size": PAGE, "write_model_s": round(write_s, 1)},
            "e2e": dict(value=round(produced / dt, 1), unit="tokens/s", ms_per_step=round(dt * 1000.0 / K, 4)),
            "clocks": clocks.summary(),
        }
    except Exception as exc:  # noqa: BLE001 - the arm reports why it could not run
        return {"impl": "reference", "unavailable": f"{type(exc).__name__}: {str(exc).splitlines()[0][:200]}"}


def run_profile_step(args) -> dict:
    """A few eager (not graph-replayed) steps of one kind, for a profiler to list kernels:
    ``--only decode`` (``--batch`` requests of ``--context`` tokens) or ``--only prefill``."""
    import torch

    from qwen3_runtime_b200.config import Qwen3Config
    from qwen3_runtime_b200.engine.batch import StepEntry
    from qwen3_runtime_b200.engine.factory import build_model, build_runtime
    from qwen3_runtime_b200.ops.cuda import CudaOps
    from qwen3_runtime_b200.weights.random_init import RandomDeviceSource, expected_tensors_for

    shape = dict(SHAPE)
    if args.layers:
        shape["num_hidden_layers"] = args.layers
    cfg = Qwen3Config(**shape)
    ops = CudaOps()
    model = build_model(cfg, RandomDeviceSource(expected_tensors_for(cfg), SEED, "cuda"), dtype="bfloat16", ops=ops)
    tokens = args.batch * (args.context + args.steps + args.warmup + 64) + PREFILL_TOKENS
    rt = build_runtime(model, max_positions=cfg.max_position_embeddings, block_size=PAGE,
                       num_kv_blocks=-(-tokens // PAGE), max_num_seqs=args.batch, cuda_graph=args.graph)
    gen = torch.Generator().manual_seed(SEED)
    times = []
    if args.only == "decode":
        handles = []
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
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            rt.runner.run(entries)
            torch.cuda.synchronize()
            times.append((time.perf_counter() - t0) * 1e3)
    else:
        for s in range(args.warmup + args.steps):
            rc = rt.cache.open("p")
            rt.cache.reserve(rc, PREFILL_TOKENS)
            toks = torch.randint(1, 1000, (PREFILL_TOKENS,), generator=gen).tolist()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            rt.runner.run([StepEntry(rc, toks, [PREFILL_TOKENS - 1])])
            torch.cuda.synchronize()
            times.append((time.perf_counter() - t0) * 1e3)
            rt.cache.close(rc)
    return {"only": args.only, "batch": args.batch, "context": args.context, "layers": cfg.num_hidden_layers,
            "graph": args.graph, "ms_per_step_wall": [round(t, 3) for t in times[args.warmup:]]}


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--layers", type=int, default=0, help="fewer layers than the full model (0 = all 36)")
    parser.add_argument("--context", type=int, default=CONTEXT)
    parser.add_argument("--only", choices=["decode", "prefill"], default=None,
                        help="run just a few steps of one kind (for profilers); prints wall times")
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
    result = run_reference(args) if args.impl == "reference" else run_ours(args)
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
