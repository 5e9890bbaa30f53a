"""A model put together from a ModelSpec: embedding, a list of layers (blocks of parts), the schedule that says in
which order they run and which cache each run touches, final norm and head.  Nothing here knows an architecture."""
from ..errors import ConfigError
from ..parts.base import make


class Model:
    def __init__(self, spec, config=None):
        self.spec, self.config = spec, config
        self.embedding = make("embedding", spec.embedding)
        self.layers = [make("block", ls.block, prefix=ls.prefix) for ls in spec.layers]
        self.schedule = list(spec.schedule)
        self.final_norm = make("norm", spec.final_norm)
        self.head = make("head", spec.head)
        for run in self.schedule:
            if not 0 <= run.layer < len(self.layers):
                raise ConfigError(f"the schedule names layer {run.layer}, the model has {len(self.layers)}")
        self.hidden, self.vocab = spec.hidden, spec.vocab
        # A step can be replayed from a captured graph only if no part's forward() looks at host values of the batch
        # (sequence lengths, positions): parts say so themselves, and one that does not say it keeps graphs off.
        # (A part that holds parts of its own, as attention holds its position encoding, answers for them.)
        self.graph_safe = all(getattr(p, "graph_safe", False) for p in self.parts() + self.layers)

    def parts(self):
        out = [self.embedding]
        for b in self.layers:
            out += b.parts()
        return out + [self.final_norm, self.head]

    def wants(self):
        seen, out = {}, []
        for p in self.parts():
            for w in p.wants():
                if w.name in seen:
                    if seen[w.name].shape != w.shape:
                        raise ConfigError(f"two parts want {w.name} with different shapes")
                    continue
                seen[w.name] = w
                out.append(w)
        return out

    def bind(self, tensors, env):
        for p in self.parts():
            p.bind(tensors, env)

    def portion_alignment(self):
        """Portions of a prompt that do not reach its end must end at a multiple of this many positions: the least
        common multiple of what the parts ask for (`portion_alignment`, 1 when a part does not say)."""
        import math
        return math.lcm(*[max(1, int(getattr(p, "portion_alignment", 1))) for p in self.parts()])

    def cache_needs(self):
        """-> ({cache id: CacheNeed or None}, {cache id: StateNeed}) from the schedule: the run that writes a cache
        says what it holds; a run that only reads it must want the same."""
        needs, states = {}, {}
        for run in self.schedule:
            if run.cache is None:
                continue
            mixer = self.layers[run.layer].mixer
            need, state = mixer.cache_need(), mixer.state_need()
            if run.cache in needs and needs[run.cache] != need:
                raise ConfigError(f"cache {run.cache} is used by mixers that keep different things")
            needs[run.cache] = need
            if state is not None:
                states[run.cache] = state
        written = {r.cache for r in self.schedule if r.write}
        for run in self.schedule:
            if run.cache is not None and run.cache not in written:
                raise ConfigError(f"cache {run.cache} is read but no layer writes it")
        return needs, states

    def prepare(self, ctx):
        seen = set()
        for run in self.schedule:
            if run.layer not in seen:
                seen.add(run.layer)
                self.layers[run.layer].mixer.prepare(ctx)

    def forward(self, ctx):
        """Runs the step's tokens through the schedule.  -> float32 logits (n_out, vocab) at the wanted tokens."""
        import torch
        x = ctx.ws.get("residual", ctx.N, (self.hidden,), torch.float32)
        self.embedding.forward(ctx, x)
        pending = None
        for i, run in enumerate(self.schedule):
            # the norm that reads the stream after this block, for a block whose last product can prepare its input
            after = self.layers[self.schedule[i + 1].layer] if i + 1 < len(self.schedule) else None
            ctx.next_first_norm = after.first_norm() if hasattr(after, "first_norm") else None
            pending = self.layers[run.layer].forward(ctx, x, pending, run)
        if ctx.n_out == 0:
            return None
        h = self.final_norm.forward(ctx, x, pending, rows=ctx.dev("want"))
        return self.head.forward(ctx, h)
