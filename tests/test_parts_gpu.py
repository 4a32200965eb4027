"""Parts alone and their generality, on the GPU with the kernels, float32 and bfloat16."""

import pytest

import part_cases as pc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from qwen3_runtime_b200.ops.cuda import CudaOps

    return CudaOps()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", [pc.case_norm_part, pc.case_position_part, pc.case_mixer_part,
                                  pc.case_feed_forward_part, pc.case_run_order_layer_twice_and_shared_cache,
                                  pc.case_window_attention, pc.case_toy_state_mixer,
                                  pc.case_toy_routed_feed_forward, pc.case_toy_position_encoding,
                                  pc.case_partial_sums, pc.case_toy_state_mixer_in_captured_steps,
                                  pc.case_interleaved_pairs_biases_and_capped_logits],
                         ids=lambda f: f.__name__[5:])
def test_part(ops, case, dtype):
    case(dtype, ops, "cuda")
