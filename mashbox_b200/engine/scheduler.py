"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes, finishes and frees.

Every live request is a list of tokens (prompt + what it generated) of which the first `computed` are in the cache.
A step feeds each chosen request its next tokens: ONE token when only the last is missing (decoding), else a portion of
at most `chunk` tokens.  Decoding requests come first and always get their token; what is left of the step's token
budget goes to prompt portions, first come first served, then to new admissions.  The logits of a request are wanted
only at the step that feeds its last known token; the token sampled there is appended (mashbox-labs/mashbox schedules
the same way, one decode call for all decoding rows and at most one prefill chunk per prefilling row inside a token
budget, src/mashbox/runtime/engine.py:953-1074, on whole-context slots instead of pages).

When pages run out: a decoding request that needs a page none is free for makes the scheduler PREEMPT the most recently
admitted running request (possibly itself): its pages, row and state slot are given back, it returns to the FRONT of
the waiting queue with prompt + generated as the tokens to recompute, and its sampling continues at the same token
index, so its answer does not change.  A prompt portion never preempts a decoding request: it shrinks to the pages that
are free or waits.  A waiting request is admitted only when the pages for all its known tokens plus one are free AFTER
the pages that running prompts still have to take are set aside (window groups count only what a window and one
portion reach), so prompts that are read side by side can all be read to their end.  Should nothing be able to run
all the same while requests are live, the newest running request is preempted until something can.  A request whose
prompt + max_new can never fit the pool or the context is refused at check() and touches nothing.

Portions may have to end on a grid: `align` > 1 (a mixer that works on blocks of that many positions; the reference
cuts on multiples of 64 for such a mixer, src/mashbox/runtime/engine.py:76, 966-967) makes every portion that does not
reach the request's last known token end at a position that is a multiple of `align`.

Finish reasons as the reference (engine.py:820-827, 1040-1050): "stop" (a stop token, not emitted), "length" (max_new
reached; the first token counts), "cancel", "error".
"""
from collections import deque
from dataclasses import dataclass, field

from ..errors import RequestError
from ..sampling.params import I32_MAX, SamplingParams, check_settings, make_params


@dataclass
class Request:
    rid: object
    prompt: list
    max_new: int
    sampling: SamplingParams = field(default_factory=SamplingParams)
    stop_ids: frozenset = frozenset()
    generated: list = field(default_factory=list)
    lh: list = field(default_factory=list)      # with tracing on: (hash of the logits, top-2 gap) per generated token
    computed: int = 0
    finish: str = None
    error: str = None
    order: int = 0
    preemptions: int = 0
    needs_penalty_start: bool = True
    t_admit: float = None
    t_first: float = None
    t_end: float = None

    @property
    def tokens(self):
        return self.prompt + self.generated

    @property
    def remaining(self):
        return len(self.prompt) + len(self.generated) - self.computed


@dataclass
class Planned:
    request: Request
    start: int
    count: int
    sample: bool            # the portion ends at the request's last known token: its logits are wanted


class Scheduler:
    def __init__(self, cache, vocab, max_tokens_per_step=2048, chunk=2048, align=1):
        self.cache, self.vocab = cache, int(vocab)
        self.budget, self.chunk, self.align = int(max_tokens_per_step), int(chunk), max(1, int(align))
        if self.align > min(self.budget, self.chunk):
            raise RequestError(f"portions end on multiples of {self.align}: the step's token budget ({self.budget}) and "
                               f"the chunk ({self.chunk}) must be at least that")
        self.waiting, self.running = deque(), []
        self.counter = 0
        self.stats = dict(preemptions=0, steps=0)

    # -------------------------------------------------------------------------------------------- admission
    def capacity(self):
        return min(self.cache.max_context, self.cache.num_pages * self.cache.page_size)

    def check(self, prompt, max_new, sampling=None):
        """None when the request fits this engine, else the reason (the request is refused alone)."""
        try:
            ids = list(prompt)
        except TypeError:
            return "the prompt must be 1 or more integer token ids"
        if not ids or any(isinstance(t, bool) or not isinstance(t, int) for t in ids):
            return "the prompt must be 1 or more integer token ids"
        if min(ids) < 0 or max(ids) >= self.vocab:
            return f"token ids must be 0..{self.vocab - 1}"
        if isinstance(max_new, bool) or not isinstance(max_new, int) or not 1 <= max_new <= I32_MAX:
            return f"max_new must be an integer 1..{I32_MAX}"
        if len(ids) + max_new > self.capacity():
            return f"prompt ({len(ids)} tokens) + max_new ({max_new}) is over the context of {self.capacity()}"
        return check_settings(sampling, self.vocab)

    def add(self, rid, prompt, max_new, sampling=None, stop_ids=()):
        why = self.check(prompt, max_new, sampling)
        if why is not None:
            raise RequestError(why)
        r = Request(rid, [int(t) for t in prompt], int(max_new), make_params(sampling), frozenset(stop_ids))
        self.counter += 1
        r.order = self.counter
        self.waiting.append(r)
        return r

    def busy(self):
        return bool(self.waiting or self.running)

    # -------------------------------------------------------------------------------------------- planning
    def _preempt(self, r):
        self.cache.release(r.rid)
        self.running.remove(r)
        r.computed = 0
        r.preemptions += 1
        r.needs_penalty_start = True
        self.waiting.appendleft(r)
        self.stats["preemptions"] += 1

    def plan(self):
        """-> list of Planned for the next step (empty when nothing can run).  Pages are not taken here: the step
        function takes them; this only makes sure they are there."""
        while True:
            plan = self._plan()
            if plan or not self.running:
                return plan
            # live requests, and not one token can run: the newest running request gives way until something can
            self._preempt(max(self.running, key=lambda q: q.order))

    def _cut(self, r, n):
        """the portion of at most n tokens that request r may be fed: its end lies on the grid unless it reaches the
        request's last known token (0: no cut fits, the request waits for a step with more room)"""
        if self.align == 1 or n >= r.remaining:
            return n
        return max(0, (r.computed + n) // self.align * self.align - r.computed)

    def _plan(self):
        cache = self.cache
        free = list(cache.free_pages())
        plan, used = [], 0

        def fits(r, n):
            return all(a <= b for a, b in zip(cache.pages_needed(r.rid, n), free))

        def take(r, n):
            for gi, a in enumerate(cache.pages_needed(r.rid, n)):
                free[gi] -= a

        def owed(r, n):
            """pages request r still has to take after a portion of n tokens to hold all its known tokens + 1"""
            hold = cache.pages_to_hold(len(r.prompt) + len(r.generated) + 1, self.chunk)
            return [max(0, h - have - new) for h, have, new in
                    zip(hold, cache.pages_held(r.rid), cache.pages_needed(r.rid, n))]

        # 1. every decoding request gets its token; newest running requests give way when pages are short
        decoding = [r for r in self.running if r.remaining == 1]
        for r in list(decoding):
            if r not in self.running:
                continue
            while not fits(r, 1):
                victim = max(self.running, key=lambda q: q.order)
                self._preempt(victim)
                plan = [p for p in plan if p.request is not victim]
                free = list(cache.free_pages())
                for p in plan:
                    take(p.request, p.count)
                if victim is r:
                    break
            if r in self.running:
                plan.append(Planned(r, r.computed, 1, True))
                take(r, 1)
        used = len(plan)
        # 2. portions of prompts already running, first come first served
        aside = [0] * len(free)             # pages the running prompts have still to take after this step
        for r in self.running:
            if r.remaining <= 1:
                continue
            n = self._cut(r, min(r.remaining, self.chunk, max(0, self.budget - used)))
            while n > 0 and not fits(r, n):
                n = self._cut(r, self._shrink(r, n, free))
            if n > 0:
                plan.append(Planned(r, r.computed, n, n == r.remaining))
                take(r, n)
                used += n
            aside = [a + o for a, o in zip(aside, owed(r, n))]
        # 3. new admissions, in order, while the whole of their known tokens (+1) fits beside what is set aside
        while self.waiting and used < self.budget and cache.can_admit():
            r = self.waiting[0]
            whole = len(r.prompt) + len(r.generated) + 1
            if any(p > f - a for p, f, a in zip(cache.pages_to_hold(whole, self.chunk), free, aside)):
                break
            n = self._cut(r, min(r.remaining, self.chunk, self.budget - used))
            if n == 0:
                break
            self.waiting.popleft()
            cache.admit(r.rid)
            self.running.append(r)
            plan.append(Planned(r, r.computed, n, n == r.remaining))
            take(r, n)
            used += n
            aside = [a + o for a, o in zip(aside, owed(r, n))]
        return plan

    def _shrink(self, r, n, free):
        """the largest portion under n that the free pages allow (0 when not even one token fits)"""
        cache = self.cache
        room = min(free) * cache.page_size + (-cache.get(r.rid).reserved) % cache.page_size
        return max(0, min(n - 1, room))

    # -------------------------------------------------------------------------------------------- results
    def finish(self, r, reason, error=None):
        r.finish, r.error = reason, error
        if r in self.running:
            self.running.remove(r)
            self.cache.release(r.rid)
        elif r in self.waiting:
            self.waiting.remove(r)

    def advance(self, plan, sampled):
        """After the step: plan as returned by plan(), sampled = the token of each Planned with sample=True, in
        order.  -> requests that ended."""
        ended, it = [], iter(sampled)
        for p in plan:
            r = p.request
            r.computed += p.count
            if not p.sample:
                continue
            t = int(next(it))
            if t in r.stop_ids:
                self.finish(r, "stop")
                ended.append(r)
                continue
            r.generated.append(t)
            if len(r.generated) >= r.max_new:
                self.finish(r, "length")
                ended.append(r)
        self.stats["steps"] += 1
        return ended

    def cancel(self, r):
        if r.finish is None:
            self.finish(r, "cancel")
