"""The step packer: a decode step that continues the last one is packed incrementally (only
ids, positions, lengths and grown block-table rows change); the result must be the buffer
that packing from scratch gives, step after step, also across page boundaries, windows that
release pages, a request that leaves and a request that is preempted and starts again."""

import random

import torch

from qwen3_runtime_b200.cache import CacheManager, GroupSpec
from qwen3_runtime_b200.engine.batch import BatchBuilder, StepEntry


def _pack(builder, entries, buf, fast):
    return builder.build(entries, pad_to=4, table_width=32, scratch_page=99, scratch_slot=7, device_buffer=buf,
                         all_rows=True, need_context=not fast)


def test_incremental_decode_packing_equals_packing_from_scratch():
    rng = random.Random(3)
    cache = CacheManager([GroupSpec("full"), GroupSpec("window", window=5)], 4, 64, 8)
    quick = BatchBuilder(cache, "cpu", vocab_size=1000, max_positions=512)
    fresh = BatchBuilder(cache, "cpu", vocab_size=1000, max_positions=512)
    handles = {}
    for rid, n in (("a", 7), ("b", 1), ("c", 12)):
        rc = handles[rid] = cache.open(rid)
        cache.reserve(rc, n)
        cache.commit(rc, n)
    buf_quick = torch.zeros(512, dtype=torch.int32)
    buf_fresh = torch.zeros(512, dtype=torch.int32)
    continued = 0
    for step in range(60):
        if step == 25:  # one request leaves
            cache.close(handles.pop("b"))
        if step == 40:  # one is preempted and prefilled again
            rc = handles["c"]
            cache.reset(rc)
            cache.reserve(rc, 9)
            cache.commit(rc, 9)
        entries = []
        for rc in handles.values():
            cache.reserve(rc, 1)
            entries.append(StepEntry(rc, [rng.randrange(1000)], [0]))
        before = quick._last_decode
        _pack(quick, entries, buf_quick, fast=True)
        if before is not None and quick._last_decode is before:
            continued += 1
        ctx = _pack(fresh, entries, buf_fresh, fast=False)
        assert ctx is not None
        assert torch.equal(buf_quick, buf_fresh), f"step {step}"
        for rc in handles.values():
            cache.commit(rc, 1)
        cache.check_invariants()
    assert continued >= 50, "most steps were continuations and were packed incrementally"


def test_incremental_packing_leaves_errors_to_the_full_path():
    cache = CacheManager([GroupSpec("full")], 4, 16, 4)
    builder = BatchBuilder(cache, "cpu", vocab_size=10, max_positions=64)
    rc = cache.open("a")
    cache.reserve(rc, 3)
    cache.commit(rc, 3)
    buf = torch.zeros(256, dtype=torch.int32)
    cache.reserve(rc, 1)
    _pack(builder, [StepEntry(rc, [5], [0])], buf, fast=True)
    cache.commit(rc, 1)
    cache.reserve(rc, 1)
    try:
        _pack(builder, [StepEntry(rc, [10], [0])], buf, fast=True)
    except ValueError as err:
        assert "outside the vocabulary" in str(err)
    else:
        raise AssertionError("a token id outside the vocabulary must be refused")
