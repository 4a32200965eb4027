"""Parts alone and their generality, on the CPU with the torch statements of the kernels."""

import part_cases as pc
from emulated_ops import TorchOps

OPS, DEV, DT = TorchOps(), "cpu", "float32"


def test_norm_part():
    pc.case_norm_part(DT, OPS, DEV)


def test_position_part():
    pc.case_position_part(DT, OPS, DEV)


def test_mixer_part():
    pc.case_mixer_part(DT, OPS, DEV)


def test_feed_forward_part():
    pc.case_feed_forward_part(DT, OPS, DEV)


def test_run_order_layer_twice_and_shared_cache():
    pc.case_run_order_layer_twice_and_shared_cache(DT, OPS, DEV)


def test_window_attention():
    pc.case_window_attention(DT, OPS, DEV)


def test_toy_state_mixer_registers_builds_and_steps():
    pc.case_toy_state_mixer(DT, OPS, DEV)


def test_toy_routed_feed_forward_registers_builds_and_steps():
    pc.case_toy_routed_feed_forward(DT, OPS, DEV)


def test_toy_position_encoding_registers_builds_and_steps():
    pc.case_toy_position_encoding(DT, OPS, DEV)


def test_partial_sums_are_allowed_by_the_run_order_and_added_by_the_norm():
    pc.case_partial_sums(DT, OPS, DEV)


def test_interleaved_pairs_biases_and_capped_logits():
    pc.case_interleaved_pairs_biases_and_capped_logits(DT, OPS, DEV)
