"""The kernel table's host-side rules (no kernel runs): how many slices decode attention cuts a
sequence into, and which tcgen05 kernel a fused SwiGLU product goes to."""

import random

from qwen3_runtime_b200.ops.cuda import CudaOps


class Table:
    """What the rules read from a kernel table of a B200."""

    DECODE_BLOCKS_PER_SM = 3
    SM_COUNT = 148
    _slices_cache: dict = {}
    decode_splits = CudaOps.decode_splits


def slices(num_seqs, kv_heads, longest, head_dim=128, total=None):
    return Table().decode_splits(num_seqs, kv_heads, longest, head_dim, total_kv_len=total)


def test_slice_counts_of_decode_attention():
    # few sequences: many slices, until every block slot (3 x 148) has a block
    assert slices(1, 8, 4096) == 16 and slices(8, 8, 4096) == 6 and slices(8, 8, 8192) == 6
    # more (sequence, kv head) pairs than slots: whole sequences while they are short, slices of about
    # a thousand keys when they are long
    assert slices(64, 8, 768) == 1 and slices(64, 8, 4096) in (4, 5) and slices(32, 8, 1024) == 1
    # never slices of less than 64 keys, and none at all for a handful of keys
    rnd = random.Random(0)
    for _ in range(2000):
        B, L, D = rnd.randint(1, 300), rnd.randint(1, 40000), rnd.choice([64, 128, 256])
        s = slices(B, rnd.choice([1, 2, 4, 8]), L, D)
        assert 1 <= s <= 64 and (s == 1 or -(-L // s) >= 33), (B, L, D, s)
    assert slices(5, 8, 63) == 1 and slices(1, 1, 1) == 1


def test_a_batch_of_mixed_lengths_counts_as_fewer_sequences_of_the_longest():
    # 48 sequences of 4096 keys fill the slots with one block per pair; when they add up to
    # half of that, the longest ones can be cut in two
    assert slices(48, 8, 4096) == 1
    assert slices(48, 8, 4096, total=24 * 4096) == 2
    assert slices(48, 8, 4096, total=48 * 4096) == 1
    # the answer for a list of lengths; a window bounds what a sequence counts for
    lens = [4096] * 3 + [100] * 45
    assert CudaOps.decode_slices_for(Table(), lens, 8, 128, None) == slices(48, 8, 4096, total=sum(lens))
    assert CudaOps.decode_slices_for(Table(), lens, 8, 128, 200) == CudaOps.decode_slices_for(
        Table(), [263] * 3 + [100] * 45, 8, 128, None)


def test_which_tcgen05_kernel_a_fused_swiglu_product_goes_to():
    plan = lambda M, I: CudaOps._tcgen05_plan(Table, M, I)  # noqa: E731
    # 1280 tokens x 9728: five token tiles of 256 on pairs; 640: five tiles of 128 on single SMs
    # (three tiles of 256 would leave a quarter of the last one and most of a fourth round empty)
    assert plan(1280, 9728)[0] and not plan(640, 9728)[0]
    pair, token_fill, share = plan(520, 9728)
    assert token_fill < CudaOps.TCGEN05_MIN_TOKEN_FILL  # 8 tokens in the last tile: the library's finer tiles win
    for M in (512, 640, 1024, 2048, 4096):
        _pair, token_fill, share = plan(M, 9728)
        assert token_fill == 1.0 and share >= CudaOps.TCGEN05_MIN_SHARE, M
    assert plan(256, 9728)[2] < CudaOps.TCGEN05_MIN_SHARE  # not even a round and a half of work
