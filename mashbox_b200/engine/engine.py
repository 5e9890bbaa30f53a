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


class _Flight:
    """A step that is queued on the GPU: its plan, the entries that sample, where each sampled token goes in its
    request's `generated`, the handle of the ids on their way to the host, and the requests that end with this step
    because they reach max_new."""

    def __init__(self, plan, picks, index, pending, ended):
        self.plan, self.picks, self.index, self.pending, self.ended = plan, picks, index, pending, ended


class Engine:
    def __init__(self, model, engine_config=None, options=None, log=None, trace=None):
        """trace: record per generated token the order-independent hash of its logits and the gap between the two
        largest (generate() then returns them under "lh"); None reads MASHBOX_TRACE=1 from the environment, as the
        reference does (src/mashbox/cli.py:1062, src/mashbox/runtime/engine.py:80-89, 253-262)."""
        import os
        self.trace = bool(trace) if trace is not None else os.environ.get("MASHBOX_TRACE") == "1"
        self.cfg = engine_config or EngineConfig()
        self.model = model
        self.runner = ModelRunner(model, self.cfg, options)
        self.cache = self.runner.cache
        align = model.portion_alignment() if hasattr(model, "portion_alignment") else 1
        self.scheduler = Scheduler(self.cache, model.vocab, self.cfg.max_tokens_per_step, self.cfg.chunk, align)
        self.sampler = Sampler(model.vocab, self.cfg.max_requests, self.runner.device)
        self.log = log
        self.counter = 0
        self._flight = None            # the step that is queued on the GPU and not booked yet
        self.stats = dict(steps=0, prompt_tokens=0, generated_tokens=0, deferred=0)

    @classmethod
    def from_folder(cls, folder, dtype="bfloat16", device="cuda:0", options=None, log=None, trace=None,
                    **engine_options):
        cfg = EngineConfig(dtype=dtype, device=device, **engine_options)
        model = load_model(folder, dtype=cfg.dtype, device=device, log=log)
        return cls(model, cfg, options, log, trace)

    @classmethod
    def from_config(cls, config, source, dtype="bfloat16", device="cuda:0", options=None, log=None, trace=None,
                    **engine_options):
        """config: an architecture's typed configuration; source: a TensorSource with its tensors (for instance
        weights.random_init.RandomSource)."""
        from .. import ops
        from .loading import build_model
        cfg = EngineConfig(dtype=dtype, device=device, **engine_options)
        model = build_model(config.to_hf(), source, cfg.dtype, device, ops=ops, log=log)
        return cls(model, cfg, options, log, trace)

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
        return self.scheduler.busy() or self._flight is not None

    def cancel(self, rows):
        for r in rows:
            if r.finish is not None:
                continue
            self.scheduler.cancel(r)
            while r.generated and r.generated[-1] == self.PLACEHOLDER:      # tokens of steps still in flight: dropped
                r.generated.pop()

    PLACEHOLDER = -1        # stands for a token that is being sampled while the next step is prepared and queued

    def _prepare(self, before=None):
        """Plans the next step and lays its arrays out on the host.  -> (plan, entries, ctx), None when nothing is
        left to run, or DEFER.  before: the step still in flight; a request's token that it is sampling stands in the
        request as a placeholder, and the plan says where the device has to fill it in.  DEFER: this step cannot be
        laid out before those ids are on the host (a penalty state would have to be rebuilt from them)."""
        plan = self.scheduler.plan()
        if not plan:
            if self.scheduler.busy():
                raise RequestError("the scheduler has requests but nothing can run (the cache pool is too small)")
            return None
        source = {id(p.request): j for j, p in enumerate(before.picks)} if before is not None else {}
        entries, patches, at = [], [], 0
        for p in plan:
            r = p.request
            tokens = r.tokens[p.start:p.start + p.count]
            last = len(r.prompt) + len(r.generated) - 1
            if r.generated and r.generated[-1] == self.PLACEHOLDER:
                if p.sample and r.sampling.penalised and r.needs_penalty_start:
                    self.stats["deferred"] += 1
                    return self.DEFER
                if p.start <= last < p.start + p.count:
                    patches.append((at + last - p.start, source[id(r)]))
            entries.append((r.rid, tokens, [p.count - 1] if p.sample else []))
            at += p.count
        # the sampler's settings of the rows that sample go to the device with the step's arrays
        rows = [(p.request.sampling, len(p.request.generated), self.cache.get(p.request.rid).state_slot)
                for p in plan if p.sample]
        packed = self.sampler.pack(rows) if rows else None
        ctx = self.runner.prepare(entries, patches, {"sample_rows": packed} if packed is not None else None)
        return plan, entries, ctx, rows

    DEFER = "defer"

    def _launch(self, prep, before=None):
        """Queues a prepared step and its sampling, and books it with a placeholder for every token being sampled.
        -> the step in flight."""
        plan, entries, ctx, rows = prep
        logits = self.runner.launch(ctx, entries, self.sampler.ret if before is not None else None)
        picks = [p for p in plan if p.sample]
        for p, (_, _, slot) in zip(picks, rows):
            r = p.request
            if r.sampling.penalised and r.needs_penalty_start:
                self.sampler.start_row(slot, r.prompt, r.generated)
            r.needs_penalty_start = False
        params = self.runner.inputs.get("sample_rows") if self.runner.inputs.has("sample_rows") else None
        pending = self.sampler.sample_async(logits, rows, self.runner.err, params, trace=self.trace)
        ended = self.scheduler.advance(plan, [self.PLACEHOLDER] * len(picks))
        return _Flight(plan, picks, [len(p.request.generated) - 1 for p in picks], pending, ended)

    def step(self):
        """One scheduler step: one batched model step, sampling, bookkeeping.  -> requests that ended.

        Two steps are in flight at a time.  A step is queued (model, sampling, the copy of the ids to the host) and
        booked with a placeholder for every token being sampled; the next step is planned and laid out from that state
        and queued as well -- the device copies the sampled ids into its input tokens -- and only then does the host
        wait for the ids of the first, book them and return.  So the GPU never waits for the host between steps.  What
        a placeholder cannot foresee is a stop token: the request then ends as it should, one step late for the GPU:
        the step already queued carries a token of it whose result is dropped."""
        cur = nxt = None
        try:
            if self._flight is None:
                prep = self._prepare()
                if prep is None:
                    return []
                self._flight = self._launch(prep)
            cur = self._flight
            if self.scheduler.busy():
                prep = self._prepare(cur)
                if prep is not None and prep is not self.DEFER:
                    nxt = self._launch(prep, cur)
            tokens = self.sampler.wait(cur.pending)
        except BaseException as e:
            self._flight = None
            self._drop_live([f for f in (cur, nxt) if f is not None], f"a step failed: {type(e).__name__}: {e}")
            raise
        self._flight = nxt
        now = time.perf_counter()
        ended = list(cur.ended)
        traced = self.sampler.trace_of(cur.pending) if self.trace and cur.pending is not None else None
        for j, (p, i, t) in enumerate(zip(cur.picks, cur.index, tokens)):
            r = p.request
            if r.finish not in (None, "length") or i >= len(r.generated):
                continue                        # cancelled or stopped since the step was queued: the token is dropped
            if r.t_first is None:
                r.t_first = now
            if t in r.stop_ids:                 # the stop token is not emitted; the request ends here
                del r.generated[i:]             # its placeholder, and that of the step queued after it
                if r.finish is None:
                    self.scheduler.finish(r, "stop")
                    ended.append(r)
                else:
                    r.finish = "stop"           # it had also reached max_new: the stop token wins, as in the reference
                continue
            r.generated[i] = t
            if traced is not None:
                r.lh.append(traced[j])
        for r in ended:
            r.t_end = now
        self.stats["steps"] += 1
        self.stats["prompt_tokens"] += sum(p.count for p in cur.plan if p.count > 1 or not p.sample)
        self.stats["generated_tokens"] += len(tokens)
        return ended

    def _drop_live(self, flights=(), why="a step failed"):
        """After a failed step nothing that was live can be trusted: every live request ends with "error" and the
        cache is given back whole (the reference drops its live rows the same way, engine.py:752-762).  flights: the
        steps that were queued and never booked; the tokens they stood placeholders for never arrive, so the
        placeholders go, and a request that had reached max_new on such a placeholder ends with "error" too."""
        for f in flights:
            for p in f.picks:
                r = p.request
                had = False
                while r.generated and r.generated[-1] == self.PLACEHOLDER:
                    r.generated.pop()
                    had = True
                if had and r.finish == "length":
                    r.finish, r.error = "error", why
        for r in list(self.scheduler.running) + list(self.scheduler.waiting):
            try:
                self.scheduler.finish(r, "error", why)
            except Exception:
                pass

    # -------------------------------------------------------------------------------------------- generate
    def generate(self, prompts, max_new=128, stop_ids=(), samp=None, on_step=None):
        """prompts: lists of token ids.  -> dict(ids, finish, timing{prefill_s, decode_s, decode_calls, new_tokens,
        sampled}[, lh]).  on_step(ids, finish) is called after every step and may return indexes of prompts to cancel."""
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
                seen = [r.generated[:-1] if r.generated and r.generated[-1] == self.PLACEHOLDER else r.generated
                        for r in rows]
                self.cancel([rows[i] for i in on_step(seen, [r.finish for r in rows]) or ()])
        t2 = time.perf_counter()
        t1 = max([r.t_first for r in rows if r.t_first is not None] or [t2])
        out = dict(ids=[list(r.generated) for r in rows], finish=[r.finish for r in rows],
                   preemptions=[r.preemptions for r in rows],
                   timing=dict(prefill_s=t1 - t0, decode_s=t2 - t1, decode_calls=calls,
                               new_tokens=sum(len(r.generated) for r in rows),
                               sampled=any(not r.sampling.greedy for r in rows)))
        if self.trace:
            out["lh"] = [list(r.lh) for r in rows]         # (hash, top-2 gap) per generated token
        return out
