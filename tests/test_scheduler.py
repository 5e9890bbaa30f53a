"""-m "not gpu": the scheduler's decisions, with the cache manager on the host and a scripted step."""
import random

import pytest

from mashbox_b200.cache.manager import CacheManager, CacheNeed
from mashbox_b200.engine.scheduler import Scheduler
from mashbox_b200.errors import RequestError


def make(pages=16, page=4, requests=4, budget=16, chunk=8, vocab=100, context=0):
    cache = CacheManager({0: CacheNeed.keys_and_values(1, 16)}, {}, page, pages, requests, context)
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


def test_two_long_prompts_side_by_side_cannot_starve_each_other():
    """budget > chunk: two prompts that each fit the pool alone were once admitted together, shrank each other to
    nothing and left an empty plan.  Pages a running prompt still has to take are now set aside before anyone is let in."""
    cache, s = make(pages=25, page=4, requests=4, budget=64, chunk=32)
    a = s.add("a", list(range(80)), 4)
    b = s.add("b", list(range(60)), 4)
    steps = 0
    while s.busy():
        plan, _ = run_step(cache, s)
        assert plan, (steps, [(r.rid, r.computed) for r in s.running], cache.free_pages())
        if steps == 0:
            assert [p.request.rid for p in plan] == ["a"] and b in s.waiting      # 21 + 16 pages do not fit 25
        steps += 1
        assert steps < 100
    assert a.finish == b.finish == "length" and s.stats["preemptions"] == 0
    assert cache.free_pages() == [25]


def test_nothing_can_run_while_requests_are_live_the_newest_gives_way():
    """a state the admission rule keeps from arising is still resolved: pages taken behind the scheduler's back leave
    two running prompts with no room; the newest is preempted and the other goes on"""
    cache, s = make(pages=10, page=4, requests=4, budget=64, chunk=8)
    a = s.add("a", list(range(20)), 2)
    run_step(cache, s)
    b = s.add("b", list(range(8)), 2)
    run_step(cache, s)
    assert a in s.running and b in s.running
    cache.admit("thief")
    cache.extend("thief", cache.free_pages()[0] * 4)
    plan = s.plan()
    assert b in s.waiting and b.preemptions == 1 and [p.request.rid for p in plan] == ["a"]


def test_portions_end_on_the_grid():
    cache = CacheManager({0: CacheNeed.keys_and_values(1, 16)}, {}, 4, 64, 4, 0)
    s = Scheduler(cache, 100, max_tokens_per_step=24, chunk=20, align=8)
    a = s.add("a", list(range(43)), 2)
    b = s.add("b", list(range(11)), 2)
    seen = {"a": [], "b": []}
    while s.busy():
        plan = s.plan()
        assert plan
        for p in plan:
            seen[p.request.rid].append((p.start, p.count))
            end = p.start + p.count
            assert end % 8 == 0 or end == len(p.request.tokens), (p.request.rid, p.start, p.count)
            cache.extend(p.request.rid, p.count)
            cache.commit(p.request.rid, p.count)
        s.advance(plan, [7 for p in plan if p.sample])
    assert seen["a"][:3] == [(0, 16), (16, 16), (32, 11)]           # 20 -> 16: the cut falls back to the grid
    assert seen["b"][0] == (0, 8)                                    # 24 - 16 = 8 tokens of budget left: one block
    with pytest.raises(RequestError, match="multiples of 8"):
        Scheduler(cache, 100, max_tokens_per_step=24, chunk=4, align=8)


def test_a_window_group_is_not_charged_for_pages_it_gives_back():
    """a long prompt in a pool whose window group could never hold all of it: admitted, because behind the window the
    pages come back at every commit"""
    needs = {0: CacheNeed.keys_and_values(1, 16), 1: CacheNeed.keys_and_values(1, 16, 6)}
    cache = CacheManager(needs, {}, 4, 40, 4, 0)
    assert cache.pages_to_hold(100, 8) == [25, 5]
    s = Scheduler(cache, 100, max_tokens_per_step=8, chunk=8)
    a = s.add("a", list(range(100)), 3)
    peak = 0
    while s.busy():
        plan, _ = run_step(cache, s)
        assert plan
        peak = max(peak, 40 - cache.free_pages()[1])
    assert a.finish == "length" and peak <= 5


@pytest.mark.parametrize("seed", range(6))
def test_random_traffic_with_long_prompts_and_a_budget_over_the_chunk(seed):
    rng = random.Random(100 + seed)
    page = rng.choice([2, 4])
    cache, s = make(pages=rng.choice([12, 20, 30]), page=page, requests=rng.choice([2, 3, 5]),
                    budget=rng.choice([24, 40, 64]), chunk=rng.choice([4, 8, 16]))
    cap = s.capacity()
    reqs, steps = [], 0
    while steps < 4000 and (s.busy() or len(reqs) < 25):
        if len(reqs) < 25 and rng.random() < 0.4:
            n = rng.randrange(1, cap - 1)
            mx = rng.randrange(1, max(2, cap - n))
            reqs.append((s.add(len(reqs), [rng.randrange(100) for _ in range(n)], mx), n, mx))
        if s.busy():
            plan, _ = run_step(cache, s, token=lambda r: rng.randrange(100))
            assert plan, "the scheduler has requests but plans nothing"
        steps += 1
    assert not s.busy()
    assert all(r.finish == "length" and len(r.generated) == mx for r, n, mx in reqs)
    assert cache.free_pages() == [cache.num_pages]
