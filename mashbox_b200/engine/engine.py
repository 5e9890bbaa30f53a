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
            self.scheduler.cancel(r)

    def step(self):
        """One scheduler step: plan, one batched model step, sample, bookkeeping.  -> requests that ended."""
        plan = self.scheduler.plan()
        if not plan:
            if self.scheduler.busy():
                raise RequestError("the scheduler has requests but nothing can run (the cache pool is too small)")
            return []
        entries = [(p.request.rid, p.request.tokens[p.start:p.start + p.count], [p.count - 1] if p.sample else [])
                   for p in plan]
        try:
            logits = self.runner.step(entries)
            picks = [p for p in plan if p.sample]
            rows = []
            for p in picks:
                r = p.request
                slot = self.cache.get(r.rid).state_slot
                if r.sampling.penalised and r.needs_penalty_start:
                    self.sampler.start_row(slot, r.prompt, r.generated)
                r.needs_penalty_start = False
                rows.append((r.sampling, len(r.generated), slot))
            tokens = self.sampler.sample(logits, rows) if picks else []
            self.runner.check()
        except BaseException:
            self._drop_live()
            raise
        now = time.perf_counter()
        for p in picks:
            if p.request.t_first is None:
                p.request.t_first = now
        ended = self.scheduler.advance(plan, tokens)
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
