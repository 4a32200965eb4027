"""The kernel table's host-side rules (no kernel runs): how many slices decode attention cuts a
sequence into, and which tcgen05 kernel a fused SwiGLU product goes to."""

import random

from qwen3_runtime_b200.ops.cuda import CudaOps


class Table:
    """What the rules read from a kernel table of a B200."""

    DECODE_BLOCKS_PER_SM = CudaOps.DECODE_BLOCKS_PER_SM
    SM_COUNT = 148

    def __init__(self):
        self._slices_cache = {}

    decode_splits = CudaOps.decode_splits
    decode_slices_for = CudaOps.decode_slices_for
    _decode_slices = CudaOps._decode_slices
    _tcgen05_plan = CudaOps._tcgen05_plan


def slices(num_seqs, kv_heads, longest, head_dim=128):
    return Table().decode_splits(num_seqs, kv_heads, longest, head_dim)


def test_slice_counts_of_decode_attention():
    # few sequences: many slices, until every block slot (3 x 148) has a block
    assert slices(1, 8, 4096) == 16 and slices(8, 8, 4096) == 6 and slices(8, 8, 8192) == 6
    # more (sequence, kv head) pairs than slots: whole sequences while they are short, slices of about
    # a thousand keys when they are long
    assert slices(64, 8, 768) == 1 and slices(64, 8, 4096) in (4, 5) and slices(32, 8, 1024) == 1
    # never slices of less than 64 keys, and none at all for a handful of keys
    rnd = random.Random(0)
    for _ in range(500):
        B, L, D = rnd.randint(1, 300), rnd.randint(1, 40000), rnd.choice([64, 128, 256])
        s = slices(B, rnd.choice([1, 2, 4, 8]), L, D)
        assert 1 <= s <= 64 and (s == 1 or -(-L // s) >= 33), (B, L, D, s)
    assert slices(5, 8, 63) == 1 and slices(1, 1, 1) == 1


def test_a_batch_of_mixed_lengths_is_cut_by_its_own_block_count():
    table = Table()
    # 48 sequences of 4096 keys fill the slots with one block per pair
    assert table.decode_slices_for([4096] * 48, 8, 128, None) == 1
    # one long sequence among short ones: the long one is cut until the slots are full; the short
    # ones stay whole (the kernel gives a shorter sequence fewer slices)
    assert table.decode_slices_for([4096] + [200] * 47, 8, 128, None) == 8
    # lengths spread over 64..4096: slices of about a thousand keys
    rnd = random.Random(1)
    assert table.decode_slices_for([rnd.randint(64, 4096) for _ in range(48)], 8, 128, None) in (3, 4, 5, 6)
    # the same lengths, the same answer as for one length; a window bounds what a sequence counts for
    assert table.decode_slices_for([4100] * 8, 8, 128, None) == slices(8, 8, 4100) == 6
    lens = [4096] * 3 + [100] * 45
    assert table.decode_slices_for(lens, 8, 128, 200) == table.decode_slices_for([263] * 3 + [100] * 45, 8, 128, None)
    assert table.decode_slices_for([], 8, 128, None) == 1


def test_which_tcgen05_kernel_a_fused_swiglu_product_goes_to():
    plan = Table()._tcgen05_plan
    # 1280 tokens x 9728: five token tiles of 256 on pairs; 640: five tiles of 128 on single SMs
    # (three tiles of 256 would leave a quarter of the last one and most of a fourth round empty)
    assert plan(1280, 9728)[0] and not plan(640, 9728)[0]
    pair, token_fill, share = plan(520, 9728)
    assert token_fill < CudaOps.TCGEN05_MIN_TOKEN_FILL  # 8 tokens in the last tile: the library's finer tiles win
    for M in (512, 640, 1024, 2048, 4096):
        _pair, token_fill, share = plan(M, 9728)
        assert token_fill == 1.0 and share >= CudaOps.TCGEN05_MIN_SHARE, M
    assert plan(256, 9728)[2] < CudaOps.TCGEN05_MIN_SHARE  # not even a round and a half of work
