"""-m "not gpu": the scheduler's decisions, with the cache manager on the host and a scripted step."""
import random

import pytest

from mashbox_b200.cache.manager import CacheManager, CacheNeed
from mashbox_b200.engine.scheduler import Scheduler
from mashbox_b200.errors import RequestError


def make(pages=16, page=4, requests=4, budget=16, chunk=8, vocab=100, context=0):
    cache = CacheManager({0: CacheNeed("full", 1, 16)}, {}, page, pages, requests, context)
    return cache, Scheduler(cache, vocab, max_tokens_per_step=budget, chunk=chunk)


def run_step(cache, s, token=lambda r: 7):
    """what the engine does with a plan: take pages, commit, sample"""
    plan = s.plan()
    for p in plan:
        cache.extend(p.request.rid, p.count)
    for p in plan:
        cache.commit(p.request.rid, p.count)
    ended = s.advance(plan, [token(p.request) for p in plan if p.sample])
    cache.check()
    return plan, ended


def test_check_refuses_alone():
    cache, s = make(context=20)
    assert s.check([1, 2], 3) is None
    assert "1 or more" in s.check([], 3)
    assert "1 or more" in s.check([1.5], 3)
    assert "token ids must be 0..99" in s.check([1, 100], 3)
    assert "max_new" in s.check([1], 0)
    assert "over the context of 20" in s.check([1] * 15, 6)
    assert "top_k" in s.check([1], 3, dict(top_k=-1))
    assert "temperature" in s.check([1], 3, dict(temperature=-0.5))
    assert "finite" in s.check([1], 3, dict(top_p=float("nan")))
    with pytest.raises(RequestError):
        s.add("x", [1] * 15, 6)
    assert not s.busy() and cache.free_pages() == [16]


def test_prompt_is_cut_into_portions_under_the_budget_and_first_token_counts():
    cache, s = make(budget=16, chunk=8)
    r = s.add("a", list(range(21)), 3)
    sizes = []
    while s.busy():
        plan, _ = run_step(cache, s)
        sizes.append([(p.count, p.sample) for p in plan])
    assert sizes == [[(8, False)], [(8, False)], [(5, True)], [(1, True)], [(1, True)]]
    assert r.finish == "length" and r.generated == [7, 7, 7] and cache.free_pages() == [16]


def test_decode_comes_first_and_the_rest_of_the_budget_goes_to_prompts_in_order():
    cache, s = make(pages=32, budget=10, chunk=8)
    a = s.add("a", [1, 2, 3], 50)
    run_step(cache, s)                       # a: whole prompt, first token
    b = s.add("b", list(range(20)), 5)
    c = s.add("c", list(range(9)), 5)
    plan, _ = run_step(cache, s)
    assert [(p.request.rid, p.count) for p in plan] == [("a", 1), ("b", 8), ("c", 1)]   # 1 + 8 + 1 = the budget of 10
    plan, _ = run_step(cache, s)
    assert [(p.request.rid, p.count) for p in plan] == [("a", 1), ("b", 8), ("c", 1)]
    plan, _ = run_step(cache, s)
    assert [(p.request.rid, p.count, p.sample) for p in plan] == [("a", 1, True), ("b", 4, True), ("c", 5, False)]
    assert a.finish is None and len(a.generated) == 4 and len(b.generated) == 1 and len(c.generated) == 0


def test_stop_token_ends_without_being_emitted():
    cache, s = make()
    r = s.add("a", [1, 2], 10, stop_ids=(9,))
    toks = iter([5, 6, 9])
    while s.busy():
        run_step(cache, s, token=lambda q: next(toks))
    assert r.finish == "stop" and r.generated == [5, 6] and cache.free_pages() == [16]


def test_cancel_while_prefilling_and_while_waiting():
    cache, s = make(requests=1, budget=4, chunk=4)
    a = s.add("a", list(range(10)), 5)
    b = s.add("b", [1], 5)
    run_step(cache, s)
    assert a.computed == 4 and b in s.waiting
    s.cancel(a)
    s.cancel(b)
    assert a.finish == "cancel" and b.finish == "cancel" and not s.busy() and cache.free_pages() == [16]
    cache.check()


def test_pages_run_out_the_newest_request_is_preempted_and_recomputed_with_the_same_answer():
    def answers(pages):
        cache, s = make(pages=pages, page=4, budget=64, chunk=64)
        reqs = [s.add(i, [10 + i] * 6, 12) for i in range(3)]
        # a scripted model: the next token is a function of the request's own tokens only
        tok = lambda r: (sum(r.tokens) * 31 + len(r.tokens)) % 97
        steps = 0
        while s.busy():
            plan, _ = run_step(cache, s, tok)
            assert plan
            steps += 1
            assert steps < 500
        assert cache.free_pages() == [pages]
        return [r.generated for r in reqs], [r.preemptions for r in reqs], s.stats["preemptions"]
    roomy, pre0, n0 = answers(64)
    tight, pre1, n1 = answers(9)              # 3 requests x 18 tokens need 15 pages of 4: not all fit at once
    assert n0 == 0 and n1 > 0
    assert tight == roomy                     # preemption changes nothing in the answers
    assert pre1[0] == 0                       # the oldest request is never the victim while others run


def test_a_waiting_request_is_admitted_only_when_its_whole_prompt_fits():
    cache, s = make(pages=6, page=4, budget=64, chunk=64)
    a = s.add("a", [1] * 14, 4)               # 4 pages
    b = s.add("b", [2] * 10, 4)               # needs 3 pages for prompt + 1: does not fit beside a
    plan, _ = run_step(cache, s)
    assert [p.request.rid for p in plan] == ["a"] and b in s.waiting
    while a.finish is None:
        run_step(cache, s)
    plan, _ = run_step(cache, s)
    assert [p.request.rid for p in plan] == ["b"]


@pytest.mark.parametrize("seed", range(6))
def test_random_traffic_always_finishes_and_frees_everything(seed):
    rng = random.Random(seed)
    cache, s = make(pages=rng.choice([8, 12, 20]), page=rng.choice([2, 4]), requests=rng.choice([2, 3, 5]),
                    budget=rng.choice([6, 16, 40]), chunk=rng.choice([4, 8, 32]))
    cap = s.capacity()
    reqs, steps = [], 0
    while steps < 3000 and (s.busy() or len(reqs) < 25):
        if len(reqs) < 25 and rng.random() < 0.3:
            n = rng.randrange(1, max(2, cap // 2))
            mx = rng.randrange(1, max(2, cap - n))
            reqs.append((s.add(len(reqs), [rng.randrange(100) for _ in range(n)], mx, stop_ids=(3,)), n, mx))
        if s.busy():
            plan, _ = run_step(cache, s, token=lambda r: rng.randrange(100))
            assert plan, "the scheduler has requests but plans nothing"
            assert sum(p.count for p in plan) <= s.budget + len(plan)
            assert len({p.request.rid for p in plan}) == len(plan)
            if rng.random() < 0.03 and s.running:
                s.cancel(rng.choice(s.running))
        steps += 1
    assert not s.busy()
    for r, n, mx in reqs:
        assert r.finish in ("length", "stop", "cancel")
        assert len(r.generated) <= mx and (r.finish != "length" or len(r.generated) == mx)
        assert 3 not in r.generated
    cache.check()
    assert cache.free_pages() == [cache.num_pages] and cache.rows.n_free == cache.max_requests
