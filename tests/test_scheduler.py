"""The scheduler's decisions, with a fake step function that computes nothing.

Mirrors what qwen3-runtime tests in tests/cpu/test_scheduler.py:22-222 and
tests/invariance/test_preempt.py:10-33 (portions reserve only their own pages, budget
sharing, decode beside prefill, shrinking to free pages, preempting the youngest,
rejecting what can never fit)."""

import pytest

from qwen3_runtime_b200.cache import CacheManager, GroupSpec
from qwen3_runtime_b200.config import EngineConfig
from qwen3_runtime_b200.engine.request import Request, RequestStatus
from qwen3_runtime_b200.engine.scheduler import Scheduler


def make(num_pages=64, page=4, seqs=4, budget=16, eos=None):
    cache = CacheManager([GroupSpec("full")], page, num_pages, seqs)
    cfg = EngineConfig(block_size=page, num_kv_blocks=num_pages, max_num_seqs=seqs, max_num_batched_tokens=budget,
                       eos_token_id=eos, cuda_graph=False)
    return Scheduler(cfg, cache), cache


def run_step(sched, cache, token=7):
    """Schedule, pretend the step ran, sample ``token`` for every request that caught up."""
    reqs = sched.schedule()
    toks = []
    for r in reqs:
        caught_up = r.cache.num_computed + r.num_scheduled_tokens >= len(r.token_ids)
        cache.commit(r.cache, r.num_scheduled_tokens)
        toks.append(token if caught_up else None)
    plan = [(r.request_id, n) for r, n in zip(reqs, [r.num_scheduled_tokens for r in reqs])]
    finished = sched.postprocess(reqs, toks)
    cache.check_invariants()
    return plan, finished


def test_prompt_is_cut_into_portions_that_reserve_only_their_pages():
    sched, cache = make(budget=6)
    r = Request(list(range(1, 15)), max_tokens=2)
    sched.add(r)
    plan, _ = run_step(sched, cache)
    assert plan == [(r.request_id, 6)] and len(r.cache.tables[0]) == 2
    plan, _ = run_step(sched, cache)
    assert plan == [(r.request_id, 6)] and len(r.cache.tables[0]) == 3
    plan, _ = run_step(sched, cache)
    assert plan == [(r.request_id, 2)] and len(r.token_ids) == 15  # caught up: sampled
    plan, fin = run_step(sched, cache)
    assert plan == [(r.request_id, 1)] and fin == [r] and r.finish_reason == "length"
    assert r.status == RequestStatus.FINISHED and cache.num_free_pages == [64] and sched.is_finished()


def test_running_first_then_waiting_share_the_budget():
    sched, cache = make(budget=10)
    a, b = Request([1] * 8, max_tokens=4), Request([2] * 8, max_tokens=4)
    sched.add(a)
    sched.add(b)
    plan, _ = run_step(sched, cache)
    assert plan == [(a.request_id, 8), (b.request_id, 2)]
    plan, _ = run_step(sched, cache)  # a decodes (1 token) beside b's next portion
    assert plan == [(a.request_id, 1), (b.request_id, 6)]
    plan, _ = run_step(sched, cache)
    assert plan == [(a.request_id, 1), (b.request_id, 1)]


def test_max_num_seqs_limits_a_step_and_order_is_first_come_first_served():
    sched, cache = make(seqs=2, budget=100)
    reqs = [Request([i + 1] * 3, max_tokens=2) for i in range(3)]
    for r in reqs:
        sched.add(r)
    plan, _ = run_step(sched, cache)
    assert [p[0] for p in plan] == [reqs[0].request_id, reqs[1].request_id]
    plan, fin = run_step(sched, cache)
    assert len(fin) == 2
    plan, _ = run_step(sched, cache)
    assert [p[0] for p in plan] == [reqs[2].request_id]


def test_portion_shrinks_to_the_free_pages():
    sched, cache = make(num_pages=3, budget=100)
    a = Request([1] * 10, max_tokens=2)  # 12 tokens: 3 pages at most
    sched.add(a)
    blocker = cache.open("blocker")
    cache.reserve(blocker, 4)  # one page away
    plan, _ = run_step(sched, cache)
    assert plan == [(a.request_id, 8)]  # two free pages only
    cache.close(blocker)
    plan, _ = run_step(sched, cache)
    assert plan == [(a.request_id, 2)]


def test_a_request_that_can_never_fit_is_rejected_at_add():
    sched, _ = make(num_pages=2)
    with pytest.raises(RuntimeError, match="needs 3 KV blocks; pool has 2"):
        sched.add(Request([1] * 8, max_tokens=1))
    sched.add(Request([1] * 7, max_tokens=1))


def test_pages_run_out_youngest_running_request_is_preempted_and_recomputed():
    sched, cache = make(num_pages=4, page=4, budget=100)
    old, young = Request([1] * 7, max_tokens=6), Request([2] * 7, max_tokens=6)
    sched.add(old)
    sched.add(young)
    emitted = {old.request_id: 0, young.request_id: 0}
    for _ in range(40):
        if sched.is_finished():
            break
        before = {r.request_id: len(r.token_ids) for r in (old, young)}
        run_step(sched, cache)
        for r in (old, young):
            emitted[r.request_id] += len(r.token_ids) - before[r.request_id]
    assert sched.is_finished() and sched.num_preemptions >= 1
    assert young.num_preemptions >= 1 and old.num_preemptions == 0  # the youngest gives way
    assert emitted == {old.request_id: 6, young.request_id: 6}  # nothing sampled twice
    assert cache.num_free_pages == [4] and cache.slots.num_free == 4


def test_preempted_request_goes_to_the_front_and_keeps_its_tokens():
    sched, cache = make(num_pages=4, page=4, budget=100)
    a, b, c = Request([1] * 8, max_tokens=8), Request([2] * 8, max_tokens=4), Request([3] * 2, max_tokens=1)
    sched.add(a)
    sched.add(b)
    run_step(sched, cache)  # a and b: 8 tokens (2 pages) each, and a sampled token: pool full
    sched.add(c)
    assert len(a.token_ids) == 9 and len(b.token_ids) == 9
    # neither can take its next token: b (the youngest) is preempted, a takes a freed page, and
    # b, at the front of the queue with all its nine tokens, starts over in what is left
    plan, _ = run_step(sched, cache)
    assert sched.num_preemptions == 1 and b.num_preemptions == 1 and a.num_preemptions == 0
    assert plan == [(a.request_id, 1), (b.request_id, 4)]
    assert len(b.token_ids) == 9 and b.num_computed_tokens == 4 and c.status == RequestStatus.WAITING


def test_deadlock_on_waiting_only_raises():
    sched, cache = make(num_pages=2, page=4)
    blocker = cache.open("x")
    cache.reserve(blocker, 8)
    sched.add(Request([1] * 3, max_tokens=1))
    with pytest.raises(RuntimeError, match="exceeds the KV pool"):
        sched.schedule()


def test_finish_reasons_stop_and_length():
    sched, cache = make(eos=9)
    a = Request([1, 2], max_tokens=5, ignore_eos=False)
    b = Request([1, 2], max_tokens=5, ignore_eos=True)
    c = Request([1, 2], max_tokens=5, ignore_eos=False, stop_token_ids=(9,), min_tokens=3)
    for r in (a, b, c):
        sched.add(r)
    for _ in range(8):
        if sched.is_finished():
            break
        run_step(sched, cache, token=9)
    assert (a.finish_reason, a.num_output_tokens) == ("stop", 1)
    assert (b.finish_reason, b.num_output_tokens) == ("length", 5)  # ignore_eos is the default
    assert (c.finish_reason, c.num_output_tokens) == ("stop", 3)  # min_tokens holds the stop back


def test_abort_returns_everything():
    sched, cache = make()
    a = Request([1] * 9, max_tokens=3)
    sched.add(a)
    run_step(sched, cache)
    sched.abort(a)
    assert sched.is_finished() and cache.num_free_pages == [64] and a.finish_reason == "abort"
