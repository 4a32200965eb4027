"""Engine versus plain implementation on the GPU with the real kernels, float32 and bfloat16."""

import pytest

import engine_cases as ec

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from qwen3_runtime_b200.ops.cuda import CudaOps

    return CudaOps()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_four_schedules(tmp_path, ops, name, dtype):
    ec.case_four_schedules(tmp_path, name, dtype, ops, "cuda")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_four_schedules_long_requests(tmp_path, ops, dtype):
    """Hundreds of keys per query, many pages per request."""
    ec.case_four_schedules(tmp_path, "B", dtype, ops, "cuda", lengths=(400, 333, 257, 480))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_first_tokens(tmp_path, ops, name, dtype):
    ec.case_first_tokens(tmp_path, name, dtype, ops, "cuda")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decode(tmp_path, ops, dtype):
    ec.case_long_decode(tmp_path, "B", dtype, ops, "cuda", total=300)


@pytest.mark.parametrize("cuda_graph", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation(tmp_path, ops, name, dtype, cuda_graph):
    ec.case_greedy_generation(tmp_path, name, dtype, ops, "cuda", cuda_graph=cuda_graph)


@pytest.mark.parametrize("cuda_graph", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_running_ahead_gives_the_same_tokens_step_by_step(tmp_path, ops, name, dtype, cuda_graph):
    ec.case_run_ahead(tmp_path, name, dtype, ops, "cuda", cuda_graph=cuda_graph)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_temperature_sampling(tmp_path, ops, dtype):
    ec.case_temperature_sampling(tmp_path, "B", dtype, ops, "cuda")


@pytest.mark.parametrize("name", ["B", "C"])
def test_four_schedules_with_every_large_product_on_tcgen05(tmp_path, name):
    """The whole model with this engine's tcgen05/TMEM kernel for every product of more than 16 tokens."""
    from qwen3_runtime_b200.ops.cuda import CudaOps

    forced = CudaOps(large_gemm="tcgen05")
    ec.case_four_schedules(tmp_path, name, "bfloat16", forced, "cuda", lengths=(400, 37, 257, 150))
    forced.raise_if_kernel_error()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_running_ahead_under_random_arrivals_stops_and_aborts(tmp_path, ops, dtype):
    ran_ahead = sum(ec.case_run_ahead_random(tmp_path, "A", dtype, ops, "cuda", seed, cuda_graph=True)
                    for seed in range(6))
    assert ran_ahead > 10


# ---- head sizes 64 and 128: the split-KV decode kernel with the newest token made inside it, the
# ---- ticket merge, the weight-streaming products with partial sums, captured graphs over them

@pytest.mark.parametrize("name", ["D", "E"])
def test_four_schedules_at_head_sizes_64_and_128(tmp_path, ops, name):
    before = ops.launches
    ec.case_four_schedules(tmp_path, name, "bfloat16", ops, "cuda", lengths=(100, 37, 61, 150, 45, 83))
    assert ops.launches > before
    ops.raise_if_kernel_error()


@pytest.mark.parametrize("name", ["D", "E"])
def test_greedy_generation_at_head_sizes_64_and_128_with_graphs(tmp_path, ops, name):
    ec.case_greedy_generation(tmp_path, name, "bfloat16", ops, "cuda", cuda_graph=True)


@pytest.mark.parametrize("name", ["D", "E"])
def test_running_ahead_at_head_sizes_64_and_128_with_graphs(tmp_path, ops, name):
    """Stop tokens found one step late (the abandoned step writes keys and values into pages that
    were already returned), aborts, late arrivals, a pool so small that a request is preempted."""
    ec.case_run_ahead(tmp_path, name, "bfloat16", ops, "cuda", cuda_graph=True)


def test_running_ahead_under_random_scenarios_at_head_size_128(tmp_path, ops):
    ran_ahead = sum(ec.case_run_ahead_random(tmp_path, "E", "bfloat16", ops, "cuda", seed, cuda_graph=True)
                    for seed in range(6))
    assert ran_ahead > 10


# ---- as many live requests as the benchmark's batches: graph buckets 8..64, the streaming
# ---- kernels' variant for more than 8 tokens, 17..64-token steps, more sequences than any bucket

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("max_live,name", [(8, "E"), (12, "A"), (16, "D"), (24, "B"), (33, "E"), (48, "D"),
                                           (64, "E"), (70, "C"), (70, "E")])
def test_mixed_schedule_and_decoding_together_with_many_live_requests(tmp_path, ops, max_live, name, dtype):
    ec.case_many_live(tmp_path, name, dtype, ops, "cuda", max_live, cuda_graph=(dtype == "bfloat16"))
    ops.raise_if_kernel_error()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cuda_graph", [False, True])
@pytest.mark.parametrize("num,name", [(8, "E"), (16, "D"), (24, "A"), (33, "E"), (64, "D"), (70, "E")])
def test_greedy_generation_of_many_requests_side_by_side(tmp_path, ops, num, name, dtype, cuda_graph):
    eng = ec.case_greedy_many(tmp_path, name, dtype, ops, "cuda", num, cuda_graph=cuda_graph)
    if cuda_graph and num <= 64:
        assert eng.runner.graphs.replays > 0


@pytest.mark.parametrize("cuda_graph", [True, False])
@pytest.mark.parametrize("name", ["D", "E"])
def test_requests_of_mixed_lengths_decoding_together(tmp_path, ops, name, cuda_graph):
    """Short and long requests in one decode batch: fewer slices for the shorter ones, the slice
    count from the lengths of the moment; a captured step for every value it takes."""
    rt = ec.case_mixed_lengths_decoding_together(tmp_path, name, "bfloat16", ops, "cuda", cuda_graph=cuda_graph)
    ops.raise_if_kernel_error()
    assert not bool(ops._tickets.any()), "every ticket word is zero again"
    if cuda_graph:
        keys = list(rt.runner.graphs.captured)
        assert rt.runner.graphs.replays == 40
        counts = {dict(k[2]).popitem()[1] for k in keys}
        assert len(keys) >= 2 and len(counts) >= 2 and max(counts) > 1, f"one graph per slice count: {keys}"
