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
    want = {dt: {rid: pm.forward_logits(raw, w, toks, act_dtype=torch.bfloat16 if dt == "bfloat16" else None)
                 for rid, toks in requests.items()} for dt in ("float32", "bfloat16")}
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
