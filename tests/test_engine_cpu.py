"""Engine versus plain implementation on the CPU (kernels replaced by their torch statements):
checks batching, the cache and the scheduler.  The same cases run on the GPU with the real
kernels in tests/test_engine_gpu.py."""

import pytest
import torch

import engine_cases as ec
from emulated_ops import TorchOps

OPS, DEV = TorchOps(), "cpu"


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_four_schedules(tmp_path, name):
    ec.case_four_schedules(tmp_path, name, "float32", OPS, DEV, lengths=(70, 37, 20, 90, 45))


def test_first_tokens(tmp_path):
    ec.case_first_tokens(tmp_path, "B", "float32", OPS, DEV)


def test_long_decode(tmp_path):
    ec.case_long_decode(tmp_path, "A", "float32", OPS, DEV, total=120)


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_alone_batched_and_preempted(tmp_path, name):
    ec.case_greedy_generation(tmp_path, name, "float32", OPS, DEV)


def test_temperature_sampling(tmp_path):
    ec.case_temperature_sampling(tmp_path, "B", "float32", OPS, DEV)


def test_without_a_gpu_the_product_path_refuses_loudly():
    from qwen3_runtime_b200.ops.cuda import CudaOps, KernelsUnavailable

    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(KernelsUnavailable, match="no CPU path"):
        CudaOps()


@pytest.mark.parametrize("name", ["A", "B"])
def test_running_ahead_gives_the_same_tokens_step_by_step(tmp_path, name):
    ec.case_run_ahead(tmp_path, name, "float32", OPS, DEV)


def test_running_ahead_under_random_arrivals_stops_and_aborts(tmp_path):
    ran_ahead = sum(ec.case_run_ahead_random(tmp_path, "A", "float32", OPS, DEV, seed) for seed in range(12))
    assert ran_ahead > 20, "the scenarios were meant to let the engine run ahead now and then"
