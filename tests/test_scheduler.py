"""The scheduler's decisions (no GPU): planning under a token budget, admission by
worst-case page credits, waiting when the pool is small, refusal of what can never
run.  The first cases mirror the reference's (tests/core_tests.cpp:123-146, :1034-1052)."""
import random

import pytest

from mini_llm_runtime_b200.cache.manager import CacheManager, GroupSpec
from mini_llm_runtime_b200.engine.scheduler import AdmissionError, Request, Scheduler, schedule_batch
from mini_llm_runtime_b200.sampling.sampler import SamplingParams


def test_mixed_budget_and_decode_protection():
    plan = schedule_batch([(0, 0, 0), (1, 10, 1), (2, 10, 2)], batch_tokens=8, prefill_chunk=4)
    assert plan == [(0, 1, False), (1, 4, True), (2, 3, True)]
    assert sum(t for _, t, _ in plan) == 8


def test_prefill_first_leaves_decodes_out_while_a_prompt_is_pending():
    plan = schedule_batch([(0, 0, 0), (1, 20, 1), (2, 20, 2)], 8, 8, "prefill_first")
    assert plan == [(1, 8, True)]
    assert schedule_batch([(0, 0, 0), (3, 0, 1)], 8, 8, "prefill_first") == [(0, 1, False), (3, 1, False)]


def test_plan_orders_by_arrival_and_stops_at_the_budget():
    plan = schedule_batch([(5, 0, 9), (6, 0, 3), (7, 3, 8), (8, 100, 1)], 6, 100)
    assert plan == [(6, 1, False), (5, 1, False), (8, 4, True)]
    assert schedule_batch([(1, 0, 0), (2, 0, 1), (3, 0, 2)], 2, 1) == [(1, 1, False), (2, 1, False)]
    with pytest.raises(ValueError):
        schedule_batch([(1, 0, 0)], 0, 1)


def make(pages, page=4, requests=4, max_len=64, windows=(None,), **kw):
    cm = CacheManager([GroupSpec(w, pages) for w in windows], page_size=page, max_requests=requests, max_model_len=max_len)
    return cm, Scheduler(cm, **kw)


def simulate(cm, sched, limit=10_000):
    """Drives scheduler + cache manager as the engine does, with a fake model that
    finishes a request after max_tokens.  Returns per-step plans and finish order."""
    plans, finished = [], []
    sched.admission_order = [r.request_id for r in sched.active]
    for _ in range(limit):
        if not (sched.waiting or sched.active):
            return plans, finished
        sched.admission_order += [r.request_id for r in sched.admit(cm.open)]
        slices = sched.plan()
        assert slices, "an active set always yields a plan"
        assert sum(s.tokens for s in slices) <= sched.max_batch_tokens
        cm.prepare([s.request.slot for s in slices], [s.tokens for s in slices])   # must never raise OutOfPages
        cm.commit()
        plans.append([(s.request.request_id, s.tokens, s.is_prefill) for s in slices])
        for s in slices:
            r = s.request
            if s.is_prefill:
                r.processed += s.tokens
                if r.prefill_remaining:
                    continue
            r.generated.append(0)
            if len(r.generated) >= r.params.max_tokens:
                # The last sampled token is never fed back, so the cache holds one less.
                assert cm.length(r.slot) == len(r.prompt) + len(r.generated) - 1
                cm.close(r.slot)
                sched.release(r)
                finished.append(r.request_id)
    raise AssertionError("the simulation did not end")


def test_chunked_prefill_then_decode_then_free():
    cm, sched = make(pages=16, max_batch_tokens=8, prefill_chunk=4)
    sched.submit(Request(0, list(range(10)), SamplingParams(max_tokens=3)))
    plans, finished = simulate(cm, sched)
    assert plans == [[(0, 4, True)], [(0, 4, True)], [(0, 2, True)], [(0, 1, False)], [(0, 1, False)]]
    assert finished == [0] and cm.free_pages(0) == 16 and sched.reserved == [0] and cm.free_slots() == 4


def test_decodes_ride_along_with_a_later_prompt():
    cm, sched = make(pages=32, max_batch_tokens=8, prefill_chunk=4)
    sched.submit(Request(0, [1, 2], SamplingParams(max_tokens=6)))
    sched.submit(Request(1, list(range(9)), SamplingParams(max_tokens=2)))
    plans, _ = simulate(cm, sched)
    assert plans[0] == [(0, 2, True), (1, 4, True)]
    assert plans[1] == [(0, 1, False), (1, 4, True)]      # a mixed step: one decoded token beside a prompt portion
    assert plans[2] == [(0, 1, False), (1, 1, True)]


def test_small_pool_makes_requests_wait_and_still_finishes_all():
    # 6 pages of 4 tokens; each request needs ceil((7+5)/4) = 3 pages: two at a time.
    cm, sched = make(pages=6, max_batch_tokens=16, prefill_chunk=8)
    for i in range(5):
        sched.submit(Request(i, list(range(7)), SamplingParams(max_tokens=5)))
    sched.admit(cm.open)
    assert [r.request_id for r in sched.active] == [0, 1] and len(sched.waiting) == 3 and sched.reserved == [6]
    plans, finished = simulate(cm, sched)
    assert finished == [0, 1, 2, 3, 4]
    assert cm.free_pages(0) == 6 and sched.reserved == [0]
    assert max(len(p) for p in plans) == 2          # never more than two live


def test_requests_that_can_never_run_are_refused():
    cm, sched = make(pages=4, max_len=64, max_batch_tokens=8, prefill_chunk=8)
    with pytest.raises(AdmissionError, match="exceeds the maximum length"):
        sched.submit(Request(0, list(range(60)), SamplingParams(max_tokens=5)))
    with pytest.raises(AdmissionError, match="the pool has 4"):
        sched.submit(Request(1, list(range(20)), SamplingParams(max_tokens=5)))
    with pytest.raises(AdmissionError, match="empty"):
        sched.submit(Request(2, [], SamplingParams(max_tokens=5)))
    with pytest.raises(ValueError):
        sched.submit(Request(3, [1], SamplingParams(max_tokens=0)))
    assert not sched.waiting


def test_scheduler_limits():
    cm = CacheManager([GroupSpec(None, 4)], 4, 4, 64)
    with pytest.raises(ValueError, match="at least the number of request slots"):
        Scheduler(cm, max_batch_tokens=3, prefill_chunk=1)
    with pytest.raises(ValueError, match="prefill_chunk"):
        Scheduler(cm, max_batch_tokens=8, prefill_chunk=9)


def test_younger_requests_pass_a_big_one_until_it_has_waited_long_enough():
    cm, sched = make(pages=8, max_batch_tokens=8, prefill_chunk=8, admission_reserve_steps=2)
    sched.submit(Request(0, list(range(8)), SamplingParams(max_tokens=12)))      # 5 pages
    sched.submit(Request(1, list(range(12)), SamplingParams(max_tokens=8)))      # 5 pages: does not fit beside 0
    sched.submit(Request(2, [1, 2], SamplingParams(max_tokens=2)))               # 1 page
    sched.submit(Request(3, [1, 2], SamplingParams(max_tokens=2)))
    sched.submit(Request(4, [1, 2], SamplingParams(max_tokens=2)))
    sched.submit(Request(5, [1, 2], SamplingParams(max_tokens=2)))
    sched.admit(cm.open)
    assert [r.request_id for r in sched.active] == [0, 2, 3, 4]                  # 1 is passed by, slots run out for 5
    plans, finished = simulate(cm, sched)
    assert sorted(finished) == [0, 1, 2, 3, 4, 5]
    # Once request 1 had waited more than two rounds nothing younger was admitted before it,
    # although request 5 would have fitted all along.
    assert sched.admission_order == [0, 2, 3, 4, 1, 5]


def test_window_group_needs_fewer_credits():
    cm, sched = make(pages=6, page=4, max_len=256, windows=(None, 8), max_batch_tokens=8, prefill_chunk=4)
    full, windowed = sched.worst_case_pages(100)
    assert full == 25 and windowed == cm.peak_pages(1, 100, 4) == 4
    cm2, sched2 = make(pages=30, page=4, max_len=256, windows=(None, 8), max_batch_tokens=8, prefill_chunk=4)
    sched2.submit(Request(0, list(range(90)), SamplingParams(max_tokens=10)))
    simulate(cm2, sched2)
    assert cm2.free_pages(0) == 30 and cm2.free_pages(1) == 30


def test_idle_pool_that_cannot_take_the_head_raises():
    cm, sched = make(pages=8, max_batch_tokens=8, prefill_chunk=8)
    sched.submit(Request(0, list(range(8)), SamplingParams(max_tokens=8)))
    sched.reserved[0] = 8       # as if credits had leaked: nothing active, nothing fits
    with pytest.raises(RuntimeError, match="no request fits an otherwise idle cache pool"):
        sched.admit(cm.open)


@pytest.mark.parametrize("seed", range(4))
def test_random_workloads_never_run_out_of_pages(seed):
    rng = random.Random(seed)
    page = rng.choice([4, 16])
    windows = (None, rng.choice([5, 20, 33]))
    cm, sched = make(pages=rng.randint(12, 30), page=page, requests=rng.randint(2, 5), max_len=160, windows=windows,
                     max_batch_tokens=rng.choice([8, 32]), prefill_chunk=rng.choice([2, 8]),
                     policy=rng.choice(["mixed", "prefill_first"]))
    n = 0
    for i in range(25):
        prompt, new = rng.randint(1, 60), rng.randint(1, 30)
        try:
            sched.submit(Request(i, list(range(prompt)), SamplingParams(max_tokens=new)))
            n += 1
        except AdmissionError:
            pass
    plans, finished = simulate(cm, sched)
    assert len(finished) == n
    assert [cm.free_pages(g) for g in range(2)] == [spec.num_pages for spec in cm.groups]
