"""The step function: one batch of (request, its next tokens) through the model, from the cache, to logits.

A step takes entries (request id, tokens, want): the request's next tokens -- a portion of its prompt of any length, or
one decoded token -- and the places among them whose logits are asked for.  All entries run as ONE batch: the tokens
are laid end to end, every kernel runs over all of them, and attention tells the sequences apart by the step's
descriptors.  Pages are taken from the cache manager before the step and the request's length is committed after it.
The scheduler, generate() and the trace replay all go through this one function.

Steps are captured in CUDA graphs, keyed by the lengths of the step's integer arrays (every launch dimension follows
from them), and replayed: the arrays live in one device buffer that is refilled before each replay.  A shape is
captured when it comes a second time -- decode batches, and the equal portions a long prompt is cut into -- and the
least recently captured graph goes when there are MAX_GRAPHS of them.  Models with a part that does not declare itself
graph_safe run without graphs.
"""
import gc
import time

import numpy as np
import torch

from .. import ops as kernels
from ..cache.manager import CacheManager
from ..errors import CacheError, RequestError
from ..parts import Env, StepContext, StepInputs, Workspace


class ModelRunner:
    MAX_GRAPHS = 64

    def __init__(self, model, engine_config, options=None):
        from .loading import torch_dtype
        self.model, self.cfg = model, engine_config
        self.options = dict(options or {})
        kernels.configure(self.options)
        self.device = torch.device(engine_config.device)
        if self.device.type != "cuda" or not torch.cuda.is_available():
            raise RequestError("mashbox_b200 runs on a CUDA device only; there is no CPU path")
        self.dtype = torch_dtype(engine_config.dtype)
        self.env = Env(self.dtype, self.device, kernels)
        needs, states = model.cache_needs()
        self.cache = CacheManager(needs, states, engine_config.page_size, engine_config.pages(),
                                  engine_config.max_requests, engine_config.max_context, self.dtype, self.device)
        self.options.setdefault("logit_rows", engine_config.max_requests)
        self.ws = Workspace(self.device, engine_config.max_tokens_per_step + engine_config.max_requests)
        self.inputs = StepInputs(self.device)
        self.err = kernels.error_word(self.device)
        self.graphs, self.seen_signatures = {}, {}
        self.use_graphs = (bool(engine_config.cuda_graphs) and not self.options.get("no_graphs", False)
                           and getattr(model, "graph_safe", False))
        self.stats = dict(steps=0, tokens=0, graph_replays=0, graph_captures=0, capture_s=0.0)
        self.capture_stream = self.graph_pool = None

    # -------------------------------------------------------------------------------------------- the step
    def step(self, entries):
        """entries: [(request id, tokens, want)] -> float32 logits (sum of wants, vocab) on the device, in the order
        of the entries and of each `want`; None when nothing is wanted.  The tensor is valid until the next step."""
        if not entries:
            return None
        return self.launch(self.prepare(entries), entries)

    def launch(self, ctx, entries, sampled=None):
        """Sends a prepared step's arrays and the changed block-table entries to the device, runs the model (a captured
        graph when the shape has come before) and commits the entries.  -> logits.  sampled: the device tensor of the
        ids sampled by the step before, for the (place, index) pairs given to prepare(): they are copied into the
        step's tokens on the device, so this step can be queued before those ids have reached the host."""
        self.inputs.upload()
        pairs = self.inputs.get("patch")
        if pairs is not None:
            if sampled is None:
                raise RequestError("the step has tokens to be filled in on the device, but no sampled ids were given")
            kernels.patch_tokens(self.inputs.get("token_ids"), sampled, pairs, pairs.numel() // 2)
        self.cache.flush_tables()
        logits = self._run_graph(ctx) if self.use_graphs else self.model.forward(ctx)
        self.commit(entries)
        return logits if logits is None or ctx.real_out == ctx.n_out else logits[:ctx.real_out]

    def begin(self, entries):
        """prepare + upload: a StepContext ready for model.forward (tests of single parts use it)"""
        ctx = self.prepare(entries)
        self.inputs.upload()
        self.cache.flush_tables()
        return ctx

    def prepare(self, entries, patches=(), extra=None):
        """Takes the pages the entries need, lays the step's integer arrays out on the host and lets the mixers plan.
        Nothing is sent to the device yet, so a step can be prepared while the step before it still runs, and token
        ids that are not known yet can be patched in on the host (patch_token) before launch(), or on the device:
        patches = (place among the step's tokens, index among the ids the step before samples) pairs.
        extra: {name: int32 array} that travel to the device with the step's own arrays (the sampler's row settings).
        -> StepContext"""
        cache = self.cache
        seen = set()
        need = [0] * len(cache.groups)
        for rid, tokens, want in entries:
            if rid in seen:
                raise RequestError(f"request {rid!r} is in the step twice")
            seen.add(rid)
            if len(tokens) < 1:
                raise RequestError(f"request {rid!r} brings no tokens")
            if any(not 0 <= int(w) < len(tokens) for w in want):
                raise RequestError(f"request {rid!r} wants a place outside its {len(tokens)} tokens")
            r = cache.get(rid)
            if r.length + len(tokens) > cache.max_context:
                raise CacheError(f"request {rid!r} would hold {r.length + len(tokens)} tokens, over the context of "
                                 f"{cache.max_context}")
            for gi, n in enumerate(cache.pages_needed(rid, len(tokens))):
                need[gi] += n
        if any(n > g.pool.n_free for n, g in zip(need, cache.groups)):
            raise CacheError("no free page")
        for rid, tokens, _ in entries:
            cache.extend(rid, len(tokens))

        S = len(entries)
        q_len = [len(t) for _, t, _ in entries]
        q_start = np.concatenate([[0], np.cumsum(q_len)[:-1]]).astype(np.int32)
        N = int(sum(q_len))
        reqs = [cache.get(rid) for rid, _, _ in entries]
        pos0 = np.asarray([r.length for r in reqs], np.int32)
        rows = np.asarray([r.row for r in reqs], np.int32)
        token_ids = np.concatenate([np.asarray(t, np.int64) for _, t, _ in entries]).astype(np.int32)
        positions = np.concatenate([p + np.arange(n, dtype=np.int32) for p, n in zip(pos0, q_len)])
        tok_row = np.repeat(rows, q_len)
        want = np.asarray([q_start[i] + int(w) for i, (_, _, ws) in enumerate(entries) for w in ws], np.int32)
        state_slots = [r.state_slot for r in reqs]
        patches = list(patches)
        real_out = len(want)

        # A decode batch is filled up to the next size of a coarse grid with sequences of one token on the cache's
        # spare page (their logits are computed and dropped), so that batches of nearby sizes are one graph.
        fill = self.filled_size(S) - S if self.use_graphs and N == S and len(want) == S else 0
        if fill > 0:
            more = np.arange(N, N + fill, dtype=np.int32)
            zeros = np.zeros(fill, np.int32)
            spare = np.full(fill, cache.spare_row, np.int32)
            token_ids, positions = np.concatenate([token_ids, zeros]), np.concatenate([positions, zeros])
            tok_row, rows = np.concatenate([tok_row, spare]), np.concatenate([rows, spare])
            want, q_start = np.concatenate([want, more]), np.concatenate([q_start, more])
            q_len, pos0 = q_len + [1] * fill, np.concatenate([pos0, zeros])
            state_slots = state_slots + [cache.spare_state_slot] * fill
            if len(patches) == S:                                    # every token of the step is filled in on the device
                patches += [(int(i), 0) for i in more]
            S, N = S + fill, N + fill

        ctx = StepContext(self.env, cache, self.ws, self.inputs, self.err, self.options)
        ctx.N, ctx.S, ctx.n_out, ctx.real_out = N, S, len(want), real_out
        ctx.rows, ctx.q_start, ctx.q_len, ctx.pos0 = rows.tolist(), q_start.tolist(), q_len, pos0.tolist()
        ctx.state_slots = state_slots
        inp = self.inputs
        inp.reset()
        inp.add("token_ids", token_ids)
        inp.add("positions", positions)
        inp.add("tok_row", tok_row)
        inp.add("want", want)
        inp.add("q_start", q_start)
        inp.add("q_len", q_len)
        inp.add("pos0", pos0)
        inp.add("seq_row", rows)
        inp.add("state_slot", ctx.state_slots)
        inp.add("patch", np.asarray([v for pair in patches for v in pair], np.int32))
        self.model.prepare(ctx)
        inp.mark()                          # what follows is read after the model has run: not part of a graph's shape
        for name, array in (extra or {}).items():
            inp.add(name, array)
        return ctx

    def filled_size(self, S):
        """the size a decode batch of S sequences is filled up to: itself up to 4, then steps of 2 up to 8, of 4 up to
        32 (16 stays a size: up to there a step runs the weight-streaming products, whose time does not depend on the
        number of tokens), of 8 up to 128, of 16 beyond; never more than the logits buffer holds"""
        if S <= 4 or not self.options.get("fill_decode_batches", True):
            return S
        step = 2 if S <= 8 else 4 if S <= 32 else 8 if S <= 128 else 16
        return max(S, min(-(-S // step) * step, int(self.options["logit_rows"])))

    def patch_token(self, index, token):
        """Sets token `index` of the prepared step (its place among the step's N tokens) before launch()."""
        self.inputs.arrays["token_ids"][index] = token

    def commit(self, entries):
        """The step's tokens are in the cache: the requests grow (and windows give pages back)."""
        for rid, tokens, _ in entries:
            self.cache.commit(rid, len(tokens))
            self.stats["tokens"] += len(tokens)
        self.stats["steps"] += 1

    def _run_graph(self, ctx):
        sig = (self.inputs.signature(), getattr(self.ws, "generation", 0), getattr(self.inputs, "generation", 0),
               kernels.scratch_generation())
        g = self.graphs.get(sig)
        if g is not None:
            g[0].replay()
            self.stats["graph_replays"] += 1
            kernels.COUNTERS["launches"] += g[2]
            return g[1]
        count = self.seen_signatures.get(sig, 0)
        self.seen_signatures[sig] = count + 1
        if count == 0:                      # first time: run eagerly (loads kernels, sizes buffers)
            return self.model.forward(ctx)
        # Captured on a stream of its own that first waits for the step's stream; the GPU goes on with the steps it
        # has queued meanwhile (no device-wide wait, no emptying of the allocator's cache).
        t0 = time.perf_counter()
        main = torch.cuda.current_stream(self.device)
        if self.capture_stream is None:
            self.capture_stream = torch.cuda.Stream(self.device)
            # One memory pool for every graph of this runner: what a library allocates while a step is captured (the
            # workspace of its matrix products) is reserved once, not once per graph.  The graphs are replayed one after
            # the other on one stream and leave nothing in the pool that anyone reads later (a step's buffers are the
            # workspace's, made outside captures), so they can share it.
            self.graph_pool = torch.cuda.graph_pool_handle()
        self.capture_stream.wait_stream(main)
        graph = torch.cuda.CUDAGraph()
        before = kernels.COUNTERS["launches"]
        # No garbage collection while the stream captures: a graph of an engine that is garbage by now (they sit in
        # reference cycles) would be destroyed in the middle of the capture, which CUDA does not permit and answers by
        # invalidating the capture.
        collecting = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.stream(self.capture_stream):
                graph.capture_begin(pool=self.graph_pool, capture_error_mode="thread_local")
                try:
                    logits = self.model.forward(ctx)
                except BaseException:
                    try:
                        graph.capture_end()
                    except Exception:
                        pass
                    raise
                graph.capture_end()
        finally:
            if collecting:
                gc.enable()
        captured = kernels.COUNTERS["launches"] - before
        main.wait_stream(self.capture_stream)
        graph.replay()
        while len(self.graphs) >= self.MAX_GRAPHS:
            self.graphs.pop(next(iter(self.graphs)))
        if len(self.seen_signatures) > 64 * self.MAX_GRAPHS:
            self.seen_signatures = {s: n for s, n in self.seen_signatures.items() if s in self.graphs}
        self.graphs[sig] = (graph, logits, captured)
        self.stats["graph_captures"] += 1
        self.stats["capture_s"] += time.perf_counter() - t0          # the host's time
        return logits

    def check(self):
        """Reads the kernels' error word (synchronises)."""
        kernels.check_error_word(self.err)
