"""The engine a user holds: a loaded model, its cache, the step function, the scheduler and the sampler.

Python entry point in the manner of mashbox-labs/mashbox's Engine (src/mashbox/runtime/engine.py:1133-1177):

    eng = Engine.from_folder(model_dir, dtype="bfloat16", max_tokens=65536)
    out = eng.generate(prompts, max_new=128, stop_ids=(), samp=None)     # prompts: lists of token ids
    out["ids"], out["finish"], out["timing"]

and for continuous batching the lower level admit(reqs) / step() / cancel(rows) / busy().  `samp[i]` is None (greedy)
or a dict(temperature, top_k, top_p, min_p, seed, repetition_penalty, frequency_penalty, presence_penalty).
"""
import time

from ..config.engine import EngineConfig
from ..errors import RequestError
from ..sampling.sampler import Sampler
from .loading import load_model
from .runner import ModelRunner
from .scheduler import Scheduler


class Engine:
    def __init__(self, model, engine_config=None, options=None, log=None):
        self.cfg = engine_config or EngineConfig()
        self.model = model
        self.runner = ModelRunner(model, self.cfg, options)
        self.cache = self.runner.cache
        self.scheduler = Scheduler(self.cache, model.vocab, self.cfg.max_tokens_per_step, self.cfg.chunk)
        self.sampler = Sampler(model.vocab, self.cfg.max_requests, self.runner.device)
        self.log = log
        self.counter = 0
        self._prepared = None          # the next step, planned and laid out while the one before it ran
        self.stats = dict(steps=0, prompt_tokens=0, generated_tokens=0)

    @classmethod
    def from_folder(cls, folder, dtype="bfloat16", device="cuda:0", options=None, log=None, **engine_options):
        cfg = EngineConfig(dtype=dtype, device=device, **engine_options)
        model = load_model(folder, dtype=cfg.dtype, device=device, log=log)
        return cls(model, cfg, options, log)

    @classmethod
    def from_config(cls, config, source, dtype="bfloat16", device="cuda:0", options=None, log=None, **engine_options):
        """config: an architecture's typed configuration; source: a TensorSource with its tensors (for instance
        weights.random_init.RandomSource)."""
        from .. import ops
        from .loading import build_model
        cfg = EngineConfig(dtype=dtype, device=device, **engine_options)
        model = build_model(config.to_hf(), source, cfg.dtype, device, ops=ops, log=log)
        return cls(model, cfg, options, log)

    # -------------------------------------------------------------------------------------------- low level
    def check(self, q):
        """None when request q = dict(ids, max_new, samp=None) fits, else the reason."""
        try:
            ids, mx = q["ids"], q["max_new"]
        except (KeyError, TypeError):
            return "ids and max_new are required"
        return self.scheduler.check(ids, mx, q.get("samp"))

    def admit(self, reqs, stop_ids=()):
        """reqs: list of dict(ids, max_new, samp=None) -> one row per request, in order.  A request that fails
        check() gets a row with finish "error" and the reason in .error, and changes nothing else."""
        from .scheduler import Request
        self._prepared = None          # a prepared step does not know the new requests
        rows = []
        for q in reqs:
            why = self.check(q)
            self.counter += 1
            if why is not None:
                r = Request(("r", self.counter), [], 0)
                r.finish, r.error = "error", why
            else:
                r = self.scheduler.add(("r", self.counter), q["ids"], q["max_new"], q.get("samp"),
                                       q.get("stop_ids", stop_ids))
                r.t_admit = time.perf_counter()
            rows.append(r)
        return rows

    def busy(self):
        return self.scheduler.busy()

    def cancel(self, rows):
        for r in rows:
            self._prepared = None
            self.scheduler.cancel(r)

    PLACEHOLDER = -1        # stands for a token that is being sampled while the next step is prepared

    def _prepare(self):
        """Plans the next step and lays its arrays out on the host.  -> (plan, entries, ctx) or None"""
        plan = self.scheduler.plan()
        if not plan:
            if self.scheduler.busy():
                raise RequestError("the scheduler has requests but nothing can run (the cache pool is too small)")
            return None
        entries = [(p.request.rid, p.request.tokens[p.start:p.start + p.count], [p.count - 1] if p.sample else [])
                   for p in plan]
        return plan, entries, self.runner.prepare(entries)

    def step(self):
        """One scheduler step: one batched model step, sampling, bookkeeping.  -> requests that ended.

        The host work of the NEXT step (planning, page bookkeeping, laying out its arrays) is done while the GPU runs
        this one: the step is booked with a placeholder for every token being sampled, the next step is prepared from
        that state, and when the sampled ids arrive they are patched into the requests and into the prepared arrays.
        A sampled stop token is the one thing the placeholder cannot foresee: the request then ends as it should and
        the prepared step is thrown away."""
        try:
            prep = self._prepared if self._prepared is not None else self._prepare()
            self._prepared = None
            if prep is None:
                return []
            plan, entries, ctx = prep
            logits = self.runner.launch(ctx, entries)
            picks = [p for p in plan if p.sample]
            rows = []
            for p in picks:
                r = p.request
                slot = self.cache.get(r.rid).state_slot
                if r.sampling.penalised and r.needs_penalty_start:
                    self.sampler.start_row(slot, r.prompt, r.generated)
                r.needs_penalty_start = False
                rows.append((r.sampling, len(r.generated), slot))
            pending = self.sampler.sample_async(logits, rows, self.runner.err)
            # book the step with placeholders and prepare the next one while the GPU works
            ended = self.scheduler.advance(plan, [self.PLACEHOLDER] * len(picks))
            nxt = self._prepare() if self.scheduler.busy() else None
            tokens = self.sampler.wait(pending)
        except BaseException:
            self._prepared = None
            self._drop_live()
            raise
        now = time.perf_counter()
        redo = False
        for p, t in zip(picks, tokens):
            r = p.request
            if r.t_first is None:
                r.t_first = now
            if t in r.stop_ids:                 # the stop token is not emitted; the request ends here
                r.generated.pop()
                if r.finish is None:
                    self.scheduler.finish(r, "stop")
                    ended.append(r)
                    redo = True                 # the prepared step still holds this request
                else:
                    r.finish = "stop"           # it had also reached max_new: the stop token wins, as in the reference
                continue
            r.generated[-1] = t
        if nxt is not None and not redo:
            nplan, nentries, nctx = nxt
            at = 0
            for p, e in zip(nplan, nentries):
                r = p.request
                last = len(r.prompt) + len(r.generated) - 1          # the place of the token sampled just now
                if p.start <= last < p.start + p.count and e[1][last - p.start] == self.PLACEHOLDER:
                    self.runner.patch_token(at + last - p.start, r.generated[-1])
                    e[1][last - p.start] = r.generated[-1]
                at += p.count
            self._prepared = nxt
        for r in ended:
            r.t_end = now
        self.stats["steps"] += 1
        self.stats["prompt_tokens"] += sum(p.count for p in plan if p.count > 1 or not p.sample)
        self.stats["generated_tokens"] += len(tokens)
        return ended

    def _drop_live(self):
        """After a failed step nothing that was live can be trusted: every live request ends with "error" and the
        cache is given back whole (the reference drops its live rows the same way, engine.py:752-762)."""
        for r in list(self.scheduler.running) + list(self.scheduler.waiting):
            try:
                self.scheduler.finish(r, "error", "a step failed")
            except Exception:
                pass

    # -------------------------------------------------------------------------------------------- generate
    def generate(self, prompts, max_new=128, stop_ids=(), samp=None, on_step=None):
        """prompts: lists of token ids.  -> dict(ids, finish, timing{prefill_s, decode_s, decode_calls, new_tokens,
        sampled}).  on_step(ids, finish) is called after every step and may return indexes of prompts to cancel."""
        n = len(prompts)
        if n < 1:
            raise ValueError("1 or more prompts per call")
        if self.busy():
            raise RuntimeError("generate() while requests are live")
        samp = list(samp or [None] * n)
        reqs = [dict(ids=list(p), max_new=max_new, samp=samp[i]) for i, p in enumerate(prompts)]
        bad = [w for w in (self.check(q) for q in reqs) if w is not None]
        if bad:
            raise ValueError(bad[0])
        t0 = time.perf_counter()
        rows = self.admit(reqs, stop_ids)
        calls = 0
        while self.busy():
            self.step()
            calls += 1
            if on_step is not None:
                self.cancel([rows[i] for i in on_step([r.generated for r in rows], [r.finish for r in rows]) or ()])
        t2 = time.perf_counter()
        t1 = max([r.t_first for r in rows if r.t_first is not None] or [t2])
        return dict(ids=[list(r.generated) for r in rows], finish=[r.finish for r in rows],
                    preemptions=[r.preemptions for r in rows],
                    timing=dict(prefill_s=t1 - t0, decode_s=t2 - t1, decode_calls=calls,
                                new_tokens=sum(len(r.generated) for r in rows),
                                sampled=any(not r.sampling.greedy for r in rows)))
