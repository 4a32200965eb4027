"""Qwen3-4B layer sizes (hidden 2560, 32/8 heads of 128, feed-forward 9728, vocabulary 151936, tied
head) with random weights and two layers: float32 logits equal the plain implementation's under
every way of cutting the work, and bfloat16 stays within its tolerance.  The kernels here run at
the sizes the benchmark uses (the tensor-core attention kernels, the weight-streaming and tcgen05
products, the 151936-wide head), which the tiny models never reach."""

import pytest
import torch

import engine_cases as ec
import plain_model as pm
from helpers import first_mismatch, peak_tokens, random_ids, run_trace, trace_mixed, trace_portions, trace_tail_decode, trace_whole
from qwen3_runtime_b200.config import Qwen3Config
from qwen3_runtime_b200.engine.factory import build_runtime, load_model
from qwen3_runtime_b200.weights import write_random_model

pytestmark = pytest.mark.gpu

CFG = Qwen3Config(vocab_size=151936, hidden_size=2560, num_hidden_layers=2, num_attention_heads=32,
                  num_key_value_heads=8, head_dim=128, intermediate_size=9728, rms_norm_eps=1e-6, rope_theta=1e6,
                  max_position_embeddings=40960, tie_word_embeddings=True)


@pytest.fixture(scope="module")
def real(tmp_path_factory):
    folder = tmp_path_factory.mktemp("qwen3_4b_shape")
    # N(0, 0.02) as in the benchmark; norm weights 1 + N(0, 0.02)
    write_random_model(CFG, folder, seed=4, std=0.02, vector_std=0.02)
    raw, w = pm.read_model_dir(folder)
    requests = {f"r{i}": random_ids(CFG.vocab_size, n, 200 + i) for i, n in enumerate((300, 70, 45))}
    w32 = {k: v.float() for k, v in w.items()}  # converted once; the plain model converts per call
    want = {dt: ec.expected_logits(raw, w32, requests, dt) for dt in ("float32", "bfloat16")}
    return folder, requests, want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_four_schedules_at_real_layer_sizes(real, dtype):
    from qwen3_runtime_b200.ops.cuda import CudaOps

    folder, requests, want = real
    ops = CudaOps()
    model, cfg, _ = load_model(folder, dtype=dtype, ops=ops)
    results = {}
    for kind, steps in (("whole", trace_whole(requests)), ("tail", trace_tail_decode(requests)),
                        ("portions", trace_portions(requests, seed=5)), ("mixed", trace_mixed(requests, seed=6))):
        rt = build_runtime(model, max_positions=cfg.max_position_embeddings, block_size=16,
                           num_kv_blocks=peak_tokens(steps, 64) // 16, max_num_seqs=4, cuda_graph=(dtype == "bfloat16"))
        results[kind] = run_trace(rt, steps, poison=True)
        ec.check_against(results[kind], want[dtype], dtype, f"4B sizes {dtype} {kind}")
    ops.raise_if_kernel_error()
    if dtype == "float32":
        whole = {rid: torch.stack([rows[p] for p in sorted(rows)]) for rid, rows in results["whole"].items()}
        for kind in ("tail", "portions", "mixed"):
            assert first_mismatch(results[kind], whole, 0.0) is None, f"{kind}: float32 logits are not bit-identical"


def _wanted_positions(steps):
    """{request: sorted positions whose logits the trace asks for}."""
    pos, out = {}, {}
    for st in steps:
        for e in st["entries"]:
            start = pos.get(e["id"], 0)
            out.setdefault(e["id"], set()).update(start + w for w in e["want"])
            pos[e["id"]] = start + len(e["tokens"])
    return {rid: sorted(p) for rid, p in out.items()}


@pytest.fixture(scope="module")
def real_fp32_weights(real):
    folder, _, _ = real
    raw, w = pm.read_model_dir(folder)
    return raw, {k: v.float() for k, v in w.items()}  # converted once; the plain model converts per call


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("max_live", [8, 33])
def test_mixed_schedule_with_many_live_requests_at_real_layer_sizes(real, real_fp32_weights, max_live, dtype):
    """Portions beside decode tokens with 8 and with 33 requests live at once: steps of a few
    tokens up to a hundred, so every range of the products' dispatch is crossed (at most 16
    tokens, 17..64, more), in a pool of exactly the peak with returned pages poisoned; then all
    of them decoding side by side through a captured graph (bfloat16)."""
    import random

    from helpers import peak_live, thin_wants
    from qwen3_runtime_b200.ops.cuda import CudaOps

    folder, _, _ = real
    raw, w32 = real_fp32_weights
    rnd = random.Random(max_live)
    requests = {f"m{i}": random_ids(CFG.vocab_size, rnd.randint(14, 40), 900 + i) for i in range(2 * max_live + 3)}
    steps = thin_wants(trace_mixed(requests, seed=9, max_live=max_live, decode_tail=4, admit=0.97))
    assert peak_live(steps) == max_live
    wanted = _wanted_positions(steps)
    rows = ec.expected_logits(raw, w32, requests, dtype, rows=wanted)
    want = ec.Expected({rid: dict(zip(wanted[rid], rows[rid])) for rid in rows})
    want.tol, want.noise = rows.tol, rows.noise
    ops = CudaOps()
    model, _cfg, _ = load_model(folder, dtype=dtype, ops=ops)
    rt = build_runtime(model, block_size=16, num_kv_blocks=peak_tokens(steps, 64) // 16, max_num_seqs=max_live,
                       cuda_graph=(dtype == "bfloat16"))
    got = run_trace(rt, steps, poison=True)
    ops.raise_if_kernel_error()
    tol = want.tol
    bad = first_mismatch(got, want, tol)
    assert bad is None, f"request {bad[0]} position {bad[1]} differs by {bad[2]:.3g} (tolerance {tol:.3g})"
    assert sum(len(v) for v in got.values()) == sum(len(v) for v in want.values())
    sizes = sorted({sum(len(e["tokens"]) for e in st["entries"]) for st in steps})
    assert sizes[0] <= 16 and (max_live < 17 or any(17 <= n <= 64 for n in sizes))


def test_a_long_prompt_takes_the_tcgen05_swiglu_product_on_the_default_path(real, real_fp32_weights):
    """A request of 1280 tokens, whole and in two portions of 640: with the default choice of
    products the fused gate_up + SwiGLU product runs on this engine's tcgen05 kernels (seen by a spy
    on the kernel table): 1280 tokens on pairs of SMs, 640 on single SMs (five tiles of 128 tokens
    fill three rounds, three tiles of 256 would leave a fourth almost empty), and the logits match
    the plain model."""
    from qwen3_runtime_b200.ops.cuda import CudaOps

    folder, _, _ = real
    raw, w32 = real_fp32_weights
    ids = random_ids(CFG.vocab_size, 1280, 77)
    positions = [0, 1, 127, 128, 300, 511, 512, 638, 639, 640, 641, 1000, 1279]
    want = pm.forward_logits(raw, w32, ids, rows=positions, act_dtype=torch.bfloat16)
    tol, _noise = ec.bf16_tolerance([want], [pm.forward_logits(raw, w32, ids, rows=positions)])
    ops = CudaOps()
    assert ops.large_gemm == "auto"
    assert ops._tcgen05_plan(1280, CFG.intermediate_size)[0] and not ops._tcgen05_plan(640, CFG.intermediate_size)[0]
    assert min(ops._tcgen05_plan(n, CFG.intermediate_size)[2] for n in (640, 1280)) >= ops.TCGEN05_MIN_SHARE
    seen = []
    real_tc = ops.linear_tcgen05

    def spy(x, weight, out=None, out_dtype=None, mode=None, pair=None):
        seen.append((x.shape[0], mode))
        return real_tc(x, weight, out=out, out_dtype=out_dtype, mode=mode, pair=pair)

    ops.linear_tcgen05 = spy
    model, _cfg, _ = load_model(folder, dtype="bfloat16", ops=ops)
    for cuts in ((1280,), (640, 640)):
        seen.clear()
        rt = build_runtime(model, block_size=16, num_kv_blocks=80, max_num_seqs=2)
        rc = rt.cache.open("long")
        rows, start = [], 0
        for n in cuts:
            rt.cache.reserve(rc, n)
            wanted = [p - start for p in positions if start <= p < start + n]
            from qwen3_runtime_b200.engine.batch import StepEntry

            rows.append(rt.runner.run([StepEntry(rc, ids[start:start + n], wanted)]).float().cpu())
            start += n
        rt.cache.close(rc)
        ops.raise_if_kernel_error()
        got = torch.cat(rows)
        assert (cuts[0], 2) in seen, f"the SwiGLU product of {cuts[0]} tokens did not reach the tcgen05 kernel: {seen}"
        assert float((got - want).abs().max()) <= tol, f"cuts {cuts}: {float((got - want).abs().max()):.3g} > {tol:.3g}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_scheduler_drives_a_model_of_real_layer_sizes(real, real_fp32_weights, dtype):
    """Six prompts through ``build_engine(...).generate_batch`` with a 256-token budget (prompts cut
    into portions that share steps with decode tokens), captured decode steps, running ahead, and
    so few pages that a request is preempted and recomputed: every generated token is, at its
    place, the plain model's argmax up to rounding."""
    from qwen3_runtime_b200.engine.factory import build_engine
    from qwen3_runtime_b200.ops.cuda import CudaOps

    folder, _, _ = real
    raw, w32 = real_fp32_weights
    # 14 pages for 672 prompt tokens: requests start as pages come free, their portions share
    # steps with decode tokens, and three times the pool is full with nobody able to go on
    prompts = [random_ids(CFG.vocab_size, n, 500 + i) for i, n in enumerate((112, 96, 128, 192, 16, 128))]
    ops = CudaOps()
    eng = build_engine(folder, dtype=dtype, ops=ops, block_size=16, num_kv_blocks=14, max_num_seqs=6,
                       max_num_batched_tokens=256, cuda_graph=True, run_ahead=True)
    got = eng.generate_batch(prompts, max_tokens=6)
    ops.raise_if_kernel_error()
    assert eng.scheduler.num_preemptions >= 2, "the pool was meant to be too small for all six"
    assert eng.cache.num_free_pages == eng.cache.num_pages
    for p, toks in zip(prompts, got):
        assert len(toks) == 6
        ec.check_greedy_within_rounding(raw, w32, p, toks, f"4B sizes {dtype}, prompt of {len(p)}", dtype=dtype)
