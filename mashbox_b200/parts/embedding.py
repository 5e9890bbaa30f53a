"""Token embedding (rows gathered into the float32 residual stream, src/mashbox/gguf/archs/dense.py:328-329) and the
output head (logits = h W^T in float32; the head is the embedding table when the model ties them, dense.py:129, 390)."""
from ..weights.loader import Want
from .base import register


class Embedding:
    graph_safe = True       # forward() depends on the batch only through the lengths of the step's arrays
    def __init__(self, vocab, hidden, name="token_embd.weight"):
        self.V, self.D, self.name = int(vocab), int(hidden), name
        self.table = None

    def wants(self):
        return [Want(self.name, (self.V, self.D), "matrix")]

    def bind(self, tensors, env):
        self.table = tensors[self.name]

    def forward(self, ctx, x):
        ctx.ops.embed(ctx.dev("token_ids"), self.table, x, ctx.err)


class LinearHead:
    graph_safe = True       # forward() depends on the batch only through the lengths of the step's arrays
    def __init__(self, vocab, hidden, tied, name="output.weight", tied_to="token_embd.weight"):
        self.V, self.D, self.tied, self.name, self.tied_to = int(vocab), int(hidden), bool(tied), name, tied_to
        self.weight = None

    def wants(self):
        return [] if self.tied else [Want(self.name, (self.V, self.D), "matrix")]

    def bind(self, tensors, env):
        self.weight = tensors[self.tied_to if self.tied else self.name]

    def forward(self, ctx, h):
        import torch
        out = ctx.ws.get("logits", h.shape[0], (self.V,), torch.float32, reserve=ctx.options.get("logit_rows", 8))
        ctx.ops.linear(h, self.weight, out=out, out_dtype=torch.float32)
        return out


register("embedding", "table", Embedding)
register("head", "linear", LinearHead)
