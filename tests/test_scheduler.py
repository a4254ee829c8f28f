"""The scheduler's decisions, with a fake step (no GPU)."""
import random

import pytest

from binfer_b200.cache import CacheManager, KVNeed
from binfer_b200.engine.scheduler import (FINISHED, Request, RequestRefused, Scheduler)
from binfer_b200.sampling import SamplingParams


def _sched(pages=16, page_size=4, max_running=4, budget=16, max_len=256):
    cache = CacheManager([KVNeed(1, 8)], page_size=page_size, num_pages=pages,
                         max_requests=max_running)
    return Scheduler(cache, max_running=max_running, max_tokens_per_step=budget,
                     max_model_len=max_len), cache


def _req(rid, n, max_tokens=4, eos=()):
    return Request(rid, list(range(1, n + 1)), SamplingParams(max_tokens=max_tokens, seed=0),
                   eos_ids=tuple(eos))


def _run(s, cache, token=lambda req: 7, limit=10_000):
    """Drive the scheduler as the engine does, with a fake model."""
    trace = []
    while s.has_work() and limit:
        limit -= 1
        plan, dropped = s.schedule()
        if not plan:
            assert dropped or not s.has_work()
            continue
        for p in plan:                                   # what the step does to the cache
            cache.reserve(p.request.rid, p.request.computed + len(p.tokens))
        for p in plan:
            cache.commit(p.request.rid, p.request.computed + len(p.tokens))
        cache.check_consistent()
        trace.append([(p.request.rid, len(p.tokens), p.sample) for p in plan])
        s.update(plan, [token(p.request) for p in plan if p.sample])
    assert limit, "the scheduler did not finish"
    return trace


def test_prompt_is_cut_into_portions_under_the_budget():
    s, cache = _sched(budget=8, pages=32)
    r = _req("a", 19, max_tokens=2)
    s.add(r)
    trace = _run(s, cache)
    assert [t[0] for t in trace] == [("a", 8, False), ("a", 8, False), ("a", 3, True), ("a", 1, True)]
    assert r.output == [7, 7] and r.finish_reason == "length" and r.state == FINISHED
    assert cache.num_free_pages() == [32]


def test_decode_comes_before_prompt_portions_and_shares_the_step():
    s, cache = _sched(budget=8, pages=64)
    a, b = _req("a", 3, max_tokens=5), _req("b", 14, max_tokens=2)
    s.add(a)
    plan, _ = s.schedule()
    assert [(p.request.rid, len(p.tokens)) for p in plan] == [("a", 3)]
    for p in plan:
        cache.reserve("a", 3); cache.commit("a", 3)
    s.update(plan, [5])
    s.add(b)
    plan, _ = s.schedule()
    # one decoded token of a, then as much of b's prompt as the budget leaves
    assert [(p.request.rid, len(p.tokens), p.sample) for p in plan] == [("a", 1, True), ("b", 7, False)]


def test_admission_is_first_come_first_served():
    s, cache = _sched(pages=6, page_size=4, budget=64, max_running=4)
    s.add(_req("big", 20, max_tokens=1))       # 5 pages + watermark
    s.add(_req("huge", 22, max_tokens=1))      # cannot fit beside big
    s.add(_req("small", 2, max_tokens=1))      # would fit, but must not jump the queue
    plan, _ = s.schedule()
    assert [p.request.rid for p in plan] == ["big"]
    assert [r.rid for r in s.waiting] == ["huge", "small"]


def test_refused_at_the_door():
    s, cache = _sched(pages=4, page_size=4, max_len=64)
    with pytest.raises(RequestRefused, match="never fit"):
        s.add(_req("x", 16))
    with pytest.raises(RequestRefused, match="max_model_len"):
        s.add(_req("y", 64))
    with pytest.raises(RequestRefused, match="empty"):
        s.add(Request("z", [], SamplingParams()))
    s.add(_req("ok", 15, max_tokens=1))


def test_stop_token_finishes_and_is_kept():
    s, cache = _sched()
    r = _req("a", 3, max_tokens=10, eos=(9,))
    s.add(r)
    toks = iter([4, 5, 9, 6])
    _run(s, cache, token=lambda req: next(toks))
    assert r.output == [4, 5, 9] and r.finish_reason == "stop"


def test_pages_run_out_last_admitted_is_preempted_and_recomputed():
    s, cache = _sched(pages=6, page_size=4, budget=64, max_running=3)
    a, b = _req("a", 7, max_tokens=12), _req("b", 7, max_tokens=12)
    s.add(a); s.add(b)
    _run(s, cache)
    assert s.num_preemptions > 0 and b.preemptions > 0 and a.preemptions == 0
    assert len(a.output) == 12 and len(b.output) == 12
    assert a.finish_reason == b.finish_reason == "length"
    assert cache.num_free_pages() == [6]


def test_lone_request_that_cannot_grow_is_finished_for_cache():
    s, cache = _sched(pages=3, page_size=4, budget=64)
    r = _req("a", 10, max_tokens=50)
    s.add(r)
    _run(s, cache)
    assert r.finish_reason == "cache" and len(r.output) == 3       # 12 tokens fill 3 pages
    assert cache.num_free_pages() == [3]


def test_max_model_len_bounds_generation():
    s, cache = _sched(pages=64, max_len=12)
    r = _req("a", 8, max_tokens=50)
    s.add(r)
    _run(s, cache)
    assert r.finish_reason == "length" and len(r.prompt) + len(r.output) == 12


@pytest.mark.parametrize("seed", range(5))
def test_random_workloads_finish_and_free_everything(seed):
    rng = random.Random(seed)
    s, cache = _sched(pages=rng.randint(8, 30), page_size=rng.choice([2, 4, 8]),
                      max_running=rng.randint(1, 4), budget=rng.choice([3, 8, 32]))
    reqs = []
    for i in range(12):
        n = rng.randint(1, 20)
        if cache.pages_for_tokens(n + 1) > cache.num_pages:
            continue
        r = _req(i, n, max_tokens=rng.randint(1, 15))
        s.add(r)
        reqs.append(r)
    _run(s, cache, token=lambda req: rng.randint(0, 50))
    for r in reqs:
        assert r.state == FINISHED and r.finish_reason in ("length", "cache")
        if r.finish_reason == "length":
            assert len(r.output) == r.params.max_tokens
    assert cache.num_free_pages() == [cache.num_pages] and not cache.requests


def test_generate_leaves_nothing_queued_when_a_prompt_is_refused():
    """A good prompt followed by an empty one: the call raises, and the good prompt does not
    stay behind to run beside the next call's requests."""
    import itertools
    from types import SimpleNamespace
    from binfer_b200.engine.engine import Engine
    eng = Engine.__new__(Engine)          # the request bookkeeping only: no device, no model
    cache = CacheManager([KVNeed(2, 16)], page_size=8, num_pages=16, max_requests=4)
    eng.scheduler = Scheduler(cache, max_running=4, max_tokens_per_step=64, max_model_len=64)
    eng.spec = SimpleNamespace(vocab_size=100, eos_token_ids=(2,))
    eng.requests, eng._ids, eng._pending = {}, itertools.count(), None
    with pytest.raises(RequestRefused):
        eng.generate([[1, 2, 3], []], max_tokens=4)
    assert not eng.scheduler.has_work() and not eng.requests
    with pytest.raises(ValueError, match="outside the vocabulary"):
        eng.generate([[1, 2, 3], [4, 100]], max_tokens=4)
    assert not eng.scheduler.has_work() and not eng.requests
