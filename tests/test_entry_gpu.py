"""The Python entry point and the command line on the GPU."""

import subprocess
import sys
from pathlib import Path

import pytest
import torch

import plain_model as pm
from engine_cases import check_greedy_within_rounding
from helpers import make_model_dir, random_ids

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_llm_generate_greedy(tmp_path, dtype):
    from qwen3_runtime_b200 import LLM, SamplingParams

    folder = make_model_dir(tmp_path, "B")
    raw, w = pm.read_model_dir(folder)
    llm = LLM(str(folder), dtype=dtype, max_num_seqs=4, max_num_batched_tokens=16, block_size=8, num_kv_blocks=64)
    prompts = [random_ids(384, n, 90 + n) for n in (5, 13, 30)]
    one = llm.generate(prompts[0], max_tokens=8)
    many = llm.generate(prompts, SamplingParams(), max_tokens=8)
    assert isinstance(one, list) and isinstance(one[0], int) and len(many) == 3
    if dtype == "float32":
        assert many == [pm.greedy_generate(raw, w, p, 8) for p in prompts] and one == many[0]
    else:
        for p, toks in zip(prompts, many):
            check_greedy_within_rounding(raw, w, p, toks, "generate")


def test_llm_without_a_model_builds_a_tiny_random_one():
    from qwen3_runtime_b200 import LLM

    llm = LLM(dtype="float32")
    out = llm.generate([1, 2, 3], max_tokens=5)
    assert len(out) == 5 and all(0 <= t < 32 for t in out)
    assert llm.generate([1, 2, 3], max_tokens=5) == out
    with pytest.raises(TypeError, match="tokenizer"):
        llm.generate("text")


def test_generation_stops_when_a_kernel_reports_an_expired_wait():
    """Kernels with bounded waits give up through a word in device memory instead of hanging.
    The test writes that word itself (nothing is made to wait): the next sampling step raises."""
    from qwen3_runtime_b200 import LLM
    from qwen3_runtime_b200.ops.cuda import KernelError

    llm = LLM(dtype="bfloat16")
    assert len(llm.generate([1, 2, 3], max_tokens=3)) == 3
    ops = llm.engine.sampler.ops
    ops._error_word(torch.device("cuda")).fill_(2)
    with pytest.raises(KernelError, match="bounded wait"):
        llm.generate([1, 2, 3], max_tokens=3)
    assert int(ops._error_word(torch.device("cuda")).item()) == 0  # reported once, then cleared
    for rid in list(llm.engine._requests):
        llm.engine.abort_request(rid)
    assert len(llm.generate([4, 5], max_tokens=2)) == 2


def test_command_line(tmp_path):
    folder = make_model_dir(tmp_path, "A")
    raw, w = pm.read_model_dir(folder)
    prompt = [5, 6, 7, 8]
    cmd = [sys.executable, "-m", "qwen3_runtime_b200.cli", "--model", str(folder), "--max-tokens", "6", "--dtype",
           "float32", "--prompt-tokens", *map(str, prompt), "--num-kv-blocks", "16", "--no-cuda-graph"]
    proc = subprocess.run(cmd, capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = dict(line.split(" ", 1) for line in proc.stdout.strip().splitlines())
    assert lines["runtime"] == str(pm.greedy_generate(raw, w, prompt, 6))
    assert lines["bytes_per_block"] == str(2 * 2 * 2 * 16 * 16 * 4) and lines["device"].startswith("cuda")
