"""The scheduler's decisions with a fake step (no GPU)."""
import random

import pytest

from kipp_b200.cache import CacheManager
from kipp_b200.engine.scheduler import Request, RequestState, Scheduler
from kipp_b200.parts.base import PagedKVSpec
from kipp_b200.sampling.params import SamplingParams

FULL = PagedKVSpec(1, 16)


def make(pages=32, page_size=4, slots=4, **kw):
    cache = CacheManager({0: FULL}, page_size, pages, slots)
    return cache, Scheduler(cache, **kw)


def fake_step(cache, plan, token_of=lambda r: 100 + len(r.output)):
    """What Engine.step does to the cache, and a made-up token per sampled entry."""
    cache.reserve([(r.id, r.fed + len(e.tokens)) for e, r in zip(plan.entries, plan.requests)])
    for e, r in zip(plan.entries, plan.requests):
        assert e.tokens == r.all_tokens[r.fed:r.fed + len(e.tokens)]     # the right tokens, in order
        cache.advance(r.id, r.fed + len(e.tokens))
    return [token_of(plan.requests[i]) for i in plan.sampled]


def run(cache, sched, **kw):
    plans = []
    while sched.has_work():
        plan = sched.schedule()
        assert plan is not None
        assert plan.tokens <= sched.max_batch_tokens
        plans.append([(e.request, len(e.tokens), list(e.want)) for e in plan.entries])
        sched.complete(plan, fake_step(cache, plan, **kw))
        cache.check()
    return plans


def test_portions_under_a_token_budget_and_decode_first():
    cache, s = make(pages=64, max_batch_tokens=16, chunk_size=10)
    s.add(Request("a", list(range(23)), 3))
    s.add(Request("b", list(range(5)), 2))
    plans = run(cache, s)
    assert plans[0] == [("a", 10, []), ("b", 5, [4])]         # budget 16: 10 + 5
    assert plans[1] == [("b", 1, [0]), ("a", 10, [])]         # b decodes first, a goes on
    assert plans[2] == [("a", 3, [2])]                        # b finished (2 tokens), a's last portion
    assert plans[3] == [("a", 1, [0])] and plans[4] == [("a", 1, [0])] and len(plans) == 5
    a, b = s.finished[1], s.finished[0]
    assert (b.id, b.output, b.finish_reason) == ("b", [100, 101], "length")
    assert (a.output, a.finish_reason) == ([100, 101, 102], "length")
    assert cache.free_pages() == [64] and cache.slots.free_slots == 4


def test_budget_splits_one_prompt_down_to_small_portions():
    cache, s = make(pages=64, max_batch_tokens=7)
    s.add(Request("a", list(range(20)), 1))
    plans = run(cache, s)
    assert [p[0][1] for p in plans] == [7, 7, 6]
    assert plans[-1][0][2] == [5]


def test_stop_token_is_not_kept_and_frees_at_once():
    cache, s = make(max_batch_tokens=64)
    s.add(Request("a", [1, 2, 3], 10, stop_token_ids=(102,)))
    run(cache, s)
    r = s.finished[0]
    assert r.output == [100, 101] and r.finish_reason == "stop" and r.state is RequestState.FINISHED
    assert cache.free_pages() == [32]


def test_fifo_admission_blocks_at_the_head():
    # 8 pages of 4: a needs 6 at most, b needs 6 -> b waits although tiny c would fit
    cache, s = make(pages=8, max_batch_tokens=64)
    s.add(Request("a", list(range(20)), 4))
    s.add(Request("b", list(range(20)), 4))
    s.add(Request("c", [1], 1))
    first = s.schedule()
    assert [r.id for r in first.requests] == ["a"]
    assert [r.id for r in s.waiting] == ["b", "c"]              # head-of-line: c stays behind b
    s.complete(first, fake_step(cache, first))
    first_seen = ["a"]
    while s.has_work():
        plan = s.schedule()
        first_seen += [r.id for r in plan.requests if r.id not in first_seen]
        s.complete(plan, fake_step(cache, plan))
    assert first_seen == ["a", "b", "c"]                        # admitted in arrival order
    assert s.stats["preemptions"] == 0


def test_reservation_never_runs_out_mid_generation():
    rng = random.Random(3)
    cache, s = make(pages=20, page_size=4, slots=4, max_batch_tokens=24, chunk_size=9)
    for i in range(12):
        s.add(Request(i, [rng.randrange(50) for _ in range(rng.randint(1, 40))], rng.randint(1, 12)))
    run(cache, s)                                               # fake_step's reserve never raises
    assert len(s.finished) == 12 and s.stats["preemptions"] == 0
    assert all(len(r.output) == r.max_new_tokens for r in s.finished)


def test_preemption_of_the_youngest_and_recompute():
    # 6 pages of 4 = 24 tokens; two requests of 8 + 8 each cannot both finish
    cache, s = make(pages=6, page_size=4, slots=4, max_batch_tokens=64, policy="preempt")
    s.add(Request("old", list(range(8)), 8))
    s.add(Request("young", list(range(10, 18)), 8))
    plans = run(cache, s)
    assert s.stats["preemptions"] >= 1
    old = next(r for r in s.finished if r.id == "old")
    young = next(r for r in s.finished if r.id == "young")
    assert old.preemptions == 0 and young.preemptions >= 1     # the oldest always proceeds
    assert len(old.output) == 8 and len(young.output) == 8
    # after the preemption the young request was fed its prompt AND what it had generated
    refeed = [p for p in plans if any(e[0] == "young" and e[1] > 8 for e in p)]
    assert refeed, plans
    assert cache.free_pages() == [6]


def test_pages_run_out_for_a_single_request_is_refused_up_front():
    cache, s = make(pages=4, page_size=4, max_batch_tokens=64)
    with pytest.raises(ValueError, match="can never fit"):
        s.add(Request("big", list(range(10)), 10))
    cache, s = make(pages=64, max_batch_tokens=64, max_positions=16)
    with pytest.raises(ValueError, match="exceeds the context"):
        s.add(Request("long", list(range(10)), 7))
    with pytest.raises(ValueError, match="top_p"):
        s.add(Request("p", [1], 1, sampling=SamplingParams(temperature=1.0, top_p=0.0)))


def test_slots_limit_running_requests():
    cache, s = make(pages=64, slots=2, max_batch_tokens=64)
    for i in range(5):
        s.add(Request(i, [1, 2, 3], 2))
    plan = s.schedule()
    assert len(plan.requests) == 2 and len(s.waiting) == 3
    s.complete(plan, fake_step(cache, plan))
    run(cache, s)
    assert [r.id for r in s.finished] == [0, 1, 2, 3, 4]


def test_window_group_reservation():
    win = PagedKVSpec(1, 16, window=8)
    cache = CacheManager({0: FULL, 1: win}, 4, {FULL: 64, win: 6}, 4)
    s = Scheduler(cache, max_batch_tokens=8, chunk_size=8)
    # 60 tokens would need 15 pages without the window; with it (8 - 1 + 8) / 4 + 1 = 5
    s.add(Request("a", list(range(50)), 10))
    run(cache, s)
    assert len(s.finished[0].output) == 10 and cache.free_pages() == [64, 6]


def test_abort_and_seeds():
    cache, s = make(max_batch_tokens=64)
    s.add(Request("a", [1, 2], 5, sampling=SamplingParams(temperature=0.5, seed=7)))
    s.add(Request("b", [1, 2], 5))
    assert s.waiting[0].rng_state == 7
    plan = s.schedule()
    s.complete(plan, fake_step(cache, plan))
    s.abort("a")
    assert cache.pages_held("b") == [1] and "a" not in cache
    run(cache, s)
    assert {r.id: r.finish_reason for r in s.finished} == {"a": "abort", "b": "length"}
