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


def test_mixed_schedule_with_twelve_live_requests(tmp_path):
    ec.case_many_live(tmp_path, "B", "float32", OPS, DEV, 12)


def test_greedy_generation_of_ten_requests_side_by_side(tmp_path):
    ec.case_greedy_many(tmp_path, "A", "float32", OPS, DEV, 10, cuda_graph=False)


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


def _tiny_engine(tmp_path, **kw):
    from helpers import TINY, make_model_dir
    from qwen3_runtime_b200.engine.factory import build_engine

    folder = make_model_dir(tmp_path, "A")
    return build_engine(folder, dtype="float32", device=DEV, ops=OPS, block_size=TINY["A"]["page_size"],
                        num_kv_blocks=40, max_num_seqs=4, max_num_batched_tokens=64, cuda_graph=False, **kw)


def test_add_request_refuses_what_no_step_could_run(tmp_path):
    """Token ids outside the vocabulary and prompts beyond the model's positions are refused when
    the request is added; a request that would outgrow the positions is cut to them and ends with
    ``length`` there, instead of failing inside a step beside other requests."""
    eng = _tiny_engine(tmp_path)
    limit = eng.runner.builder.max_positions
    assert limit == 512
    with pytest.raises(ValueError, match="outside the vocabulary"):
        eng.add_request([1, 2, 256])
    with pytest.raises(ValueError, match="outside the vocabulary"):
        eng.add_request([-1])
    with pytest.raises(ValueError, match="no room for a new token"):
        eng.add_request([1] * (limit + 1))
    assert eng.is_finished()
    other = eng.get_request(eng.add_request([3, 4, 5], max_tokens=12))
    long = eng.get_request(eng.add_request([7] * (limit - 2), max_tokens=50))
    assert long.max_tokens == 3  # positions limit-2, limit-1 take two sampled tokens; the third is never fed back
    while not eng.is_finished():
        assert eng.step()
    assert (long.finish_reason, long.num_output_tokens) == ("length", 3)
    assert (other.finish_reason, other.num_output_tokens) == ("length", 12)
    assert eng.cache.num_free_pages == eng.cache.num_pages


def test_a_failed_launch_ahead_does_not_lose_the_step_that_ran(tmp_path):
    """If putting the next decode step on the device fails, the step that is already there is
    still read: its tokens reach the requests, the error is raised afterwards, and the engine can
    go on."""
    eng = _tiny_engine(tmp_path, run_ahead=True)
    plain = _tiny_engine(tmp_path, run_ahead=False)
    prompts = [[5, 6, 7], [9, 10, 11, 12]]
    want = plain.generate_batch(prompts, max_tokens=10)
    reqs = [eng.get_request(eng.add_request(p, max_tokens=10)) for p in prompts]
    real_run = eng.runner.run
    failed = []

    def flaky(entries, device_tokens=None):
        if device_tokens is not None and not failed:
            failed.append(True)
            raise RuntimeError("injected launch failure")
        return real_run(entries, device_tokens=device_tokens)

    eng.runner.run = flaky
    raised = 0
    for _ in range(60):
        if eng.is_finished():
            break
        before = [r.num_output_tokens for r in reqs]
        try:
            eng.step()
        except RuntimeError as exc:
            assert "injected" in str(exc)
            raised += 1
            # the step that was on the device has been read all the same
            assert [r.num_output_tokens for r in reqs] == [b + 1 for b in before]
    assert raised == 1 and eng.is_finished()
    assert [r.output_token_ids for r in reqs] == want
    assert eng.cache.num_free_pages == eng.cache.num_pages
