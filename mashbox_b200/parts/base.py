"""What every part of a layer is built from: part specs, the registries of part kinds, and the step context.

A model is data: a list of LayerSpec (which block arrangement, norm, mixer and feed-forward each layer has, with every
size and constant as a parameter) and a schedule (the order layers run in).  A part kind is a class registered under a
name; the model builder looks the name up and hands the class its parameters.  No part knows which model it is in.

Interfaces (all tensors on the device; N = tokens of the step, D = the part's width):

  Norm          wants(prefix) -> [Want];  bind(tensors, env);
                forward(ctx, x, pending=None, rows=None) -> h.  x (N, D) float32 is the residual stream; pending is
                (delta, bias or None) from the sublayer before, added into x first (in place unless rows picks rows).
  Position      wants() -> [Want];  bind(tensors, env);  rotation() -> (freqs, rotary_dim, pairing) for the fused
                rotate-and-store kernel, or None with apply(ctx, qkv, heads) doing its own work in place.
  Mixer         wants(prefix);  bind;  cache_need() -> CacheNeed or None;  state_need() -> StateNeed or None;
                prepare(ctx) (host-side plan arrays into ctx.inputs, before the upload);
                forward(ctx, h, run) -> (delta (N, D), bias or None).  run says which cache id it reads and whether
                it writes it.
  FeedForward   wants(prefix);  bind;  forward(ctx, h) -> (delta, bias or None)
  Block         built from the part specs in its own PartSpec and the layer's prefix;  parts() -> every part it
                holds;  mixer: the part that owns the cache of a run;  forward(ctx, x, pending, run) -> pending

A part may set the class attribute graph_safe = True: its forward() then reads the batch from the device arrays of
ctx.inputs only, and everything it decides on the host (which kernels, how many blocks, buffer sizes) follows from the
LENGTHS of those arrays and from ctx.N, ctx.S, ctx.n_out -- never from ctx.q_len, ctx.pos0 and the other host lists,
which are for prepare().  Steps of a model whose parts all say so are captured in CUDA graphs and replayed.
"""
from dataclasses import dataclass, field

import numpy as np

from ..errors import ConfigError


class PartSpec:
    """A part kind and its parameters (sizes, constants, nested specs)."""

    def __init__(self, kind, **params):
        self.kind, self.params = kind, params

    def key(self):
        def k(v):
            return v.key() if isinstance(v, PartSpec) else (tuple(v) if isinstance(v, list) else v)
        return (self.kind,) + tuple(sorted((n, k(v)) for n, v in self.params.items()))

    def __eq__(self, other):
        return isinstance(other, PartSpec) and self.key() == other.key()

    def __hash__(self):
        return hash(self.key())

    def __repr__(self):
        return f"PartSpec({self.kind!r}, {self.params})"


@dataclass
class LayerSpec:
    """One layer: the canonical tensor-name prefix of its tensors (e.g. "blk.3.") and its block arrangement, a
    PartSpec whose parameters are the specs of the parts that arrangement puts together -- "prenorm" takes mixer, ffn
    and norm (or norm1 and norm2 when the two differ); another arrangement (post-norms, mixer and feed-forward side by
    side) is another block kind with the parts it needs."""
    prefix: str
    block: PartSpec


@dataclass(frozen=True)
class LayerRun:
    """One entry of the schedule: run layer `layer`; its mixer reads cache `cache` (None: it keeps nothing) and writes
    this step's keys and values there when `write` is set.  Two entries may name one layer (it runs twice, each time
    with the cache id its entry gives) and an entry may read a cache another layer wrote (write=False)."""
    layer: int
    cache: int = None
    write: bool = True


@dataclass
class ModelSpec:
    hidden: int
    vocab: int
    embedding: PartSpec
    layers: list
    schedule: list
    final_norm: PartSpec
    head: PartSpec


NORMS, POSITIONS, MIXERS, FEED_FORWARDS, BLOCKS, EMBEDDINGS, HEADS = {}, {}, {}, {}, {}, {}, {}
_TABLES = {"norm": NORMS, "position": POSITIONS, "mixer": MIXERS, "feed_forward": FEED_FORWARDS, "block": BLOCKS,
           "embedding": EMBEDDINGS, "head": HEADS}


def register(family, kind, cls):
    """Adds a part kind: family is norm | position | mixer | feed_forward | block | embedding | head."""
    _TABLES[family][kind] = cls
    return cls


def make(family, spec, **extra):
    table = _TABLES[family]
    if spec.kind not in table:
        raise ConfigError(f"no {family} kind {spec.kind!r} is registered (known: {', '.join(sorted(table))})")
    return table[spec.kind](**spec.params, **extra)


@dataclass
class Env:
    """Where and how a model is built: compute dtype, device, the kernels module."""
    dtype: object
    device: object
    ops: object = None


class Workspace:
    """Named device buffers that live as long as the model runner: a part asks for `rows` rows of a per-token shape
    and gets a view of a buffer made once for the largest step, so no step allocates."""

    def __init__(self, device, max_rows):
        self.device, self.max_rows, self.buffers = device, int(max_rows), {}

    def get(self, name, rows, shape, dtype, reserve=None):
        """reserve: rows to make the buffer for at first (default: the largest step); it grows when more are asked"""
        import torch
        key = (name, tuple(shape), dtype)
        buf = self.buffers.get(key)
        if buf is None or buf.shape[0] < rows:
            cap = max(rows, self.max_rows if reserve is None else reserve)
            buf = torch.empty((cap,) + tuple(shape), dtype=dtype, device=self.device)
            self.buffers[key] = buf
            self.generation = getattr(self, "generation", 0) + 1
        return buf[:rows]


class StepInputs:
    """The integer arrays of one step, packed into one pinned host buffer and sent with one copy; each array starts on
    a 16-byte boundary.  The device buffer is the same from step to step, so a captured graph finds its inputs at the
    same addresses as long as the arrays have the same lengths (the signature)."""

    STAGES = 4

    def __init__(self, device, capacity=1 << 18):
        import torch
        self.device = device
        self.hosts = [torch.empty(capacity, dtype=torch.int32).pin_memory() for _ in range(self.STAGES)] \
            if device is not None else None
        self.events = [None] * self.STAGES
        self.turn = 0
        self.dev = torch.empty(capacity, dtype=torch.int32, device=device) if device is not None else None
        self.reset()

    def reset(self):
        self.arrays, self.offsets, self.used, self.views = {}, {}, 0, {}
        self.marked = None

    def mark(self):
        """the arrays added so far are those the model reads: the signature is theirs alone"""
        self.marked = len(self.arrays)

    def add(self, name, array):
        a = np.ascontiguousarray(array, dtype=np.int32).reshape(-1)
        self.arrays[name] = a
        self.offsets[name] = self.used
        self.used += (len(a) + 3) // 4 * 4
        return name

    def has(self, name):
        return name in self.arrays

    def signature(self):
        sig = tuple((n, len(a)) for n, a in self.arrays.items())
        return sig if self.marked is None else sig[:self.marked]

    def upload(self):
        """Copies the arrays to the device buffer through one of several pinned staging buffers: a staging buffer is
        written again only after the copy that read it has run, so steps may be queued without waiting for the GPU."""
        import torch
        if self.used > self.dev.numel():
            cap = max(self.used, 2 * self.dev.numel())
            torch.cuda.synchronize(self.device)
            self.hosts = [torch.empty(cap, dtype=torch.int32).pin_memory() for _ in range(self.STAGES)]
            self.events = [None] * self.STAGES
            self.dev = torch.empty(cap, dtype=torch.int32, device=self.device)
            self.generation = getattr(self, "generation", 0) + 1
        slot = self.turn % self.STAGES
        self.turn += 1
        if self.events[slot] is not None:
            self.events[slot].synchronize()
        host = self.hosts[slot]
        hn = host.numpy()
        for n, a in self.arrays.items():
            o = self.offsets[n]
            hn[o:o + len(a)] = a
        self.dev[:self.used].copy_(host[:self.used], non_blocking=True)
        ev = self.events[slot] or torch.cuda.Event()
        ev.record()
        self.events[slot] = ev
        self.views = {n: self.dev[o:o + len(self.arrays[n])] for n, o in self.offsets.items()}

    def get(self, name):
        """device view of an array (after upload); None for an empty one"""
        v = self.views[name]
        return v if v.numel() else None

    def host_array(self, name):
        return self.arrays[name]


class StepContext:
    """Everything one step hands to the parts.  Host lists describe the batch (for parts that plan on the host),
    device arrays come from ctx.inputs after the upload.

    Per sequence of the batch (S of them): row (request row = row of the block tables), state_slot, q_start (index of
    its first token among the N tokens), q_len, pos0 (position of that first token).  Per token: token id, position,
    tok_row (request row).  want: indexes of the tokens whose logits are returned."""

    def __init__(self, env, cache, ws, inputs, err, options):
        self.env, self.ops, self.dtype, self.device = env, env.ops, env.dtype, env.device
        self.cache, self.ws, self.inputs, self.err, self.options = cache, ws, inputs, err, options
        self.N = self.S = self.n_out = self.real_out = 0
        self.rows = self.state_slots = self.q_start = self.q_len = self.pos0 = None
        self.memo = {}

    def dev(self, name):
        return self.inputs.get(name)

    # Steps of few tokens: the product that ends a sublayer adds into the residual stream itself and can leave what the
    # norm after it needs (sums of squares of the new rows by 32 columns, the new rows times that norm's weight), so the
    # next sublayer's first product needs no norm kernel.  A block names the norm that follows in `after_norm` before
    # it runs a part; the model names the first norm of the block that runs next in `next_first_norm`.
    after_norm = None
    next_first_norm = None

    def add_into_stream(self, a, w, x, bias=None):
        """x (N, D) float32 += a W^T (+ bias), in place"""
        import torch
        nxt = self.after_norm if hasattr(self.after_norm, "fusable") else None
        sums = scaled = gw = None
        if nxt is not None:
            tiles = (x.shape[1] + 31) // 32
            sums = self.ws.get("row_sums", tiles, (16,), torch.float32, reserve=tiles)
            scaled = self.ws.get("row_scaled", x.shape[0], (x.shape[1],), torch.bfloat16)
            gw = nxt.fusable()[0]
        self.memo.pop("held", None)
        if self.ops.linear_small_residual(a, w, x, bias, sums=sums, next_w=gw, scaled=scaled):
            self.memo["held"] = (x.data_ptr(), nxt, sums, scaled)

    def held_for(self, x, norm):
        """-> (sums, scaled) left for this norm by the product that last added into x, or None"""
        h = self.memo.get("held")
        return (h[2], h[3]) if h is not None and h[0] == x.data_ptr() and h[1] is norm else None

    def take_held(self, x, norm):
        h = self.held_for(x, norm)
        self.memo.pop("held", None)
        return h
