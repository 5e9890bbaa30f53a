"""RMSNorm with the residual add folded in.

y = v * rsqrt(mean(v^2) + eps) * w with the weight multiplied as stored (src/mashbox/gguf/archs/qwen35.py:343-346),
where v is the residual stream plus the output of the sublayer before (the add of src/mashbox/gguf/archs/dense.py:348,
357, here in float32).  One kernel reads x and the delta once, writes x back and writes y.
"""
from ..weights.loader import Want
from .base import register


class RMSNorm:
    graph_safe = True       # forward() depends on the batch only through the lengths of the step's arrays
    def __init__(self, width, eps, name):
        self.width, self.eps, self.name = int(width), float(eps), name
        self.weight = None

    def wants(self):
        return [Want(self.name, (self.width,), "vector")]

    def bind(self, tensors, env):
        self.weight = tensors[self.name]

    def fusable(self):
        """(weight, eps) for a product kernel that normalises the residual stream itself"""
        return self.weight, self.eps

    def forward(self, ctx, x, pending=None, rows=None):
        n_out = x.shape[0] if rows is None else rows.shape[0]
        out = ctx.ws.get("normed" if rows is None else "normed_rows", n_out, (self.width,), ctx.dtype,
                         reserve=None if rows is None else ctx.options.get("logit_rows", 8))
        delta, bias = pending if pending is not None else (None, None)
        if delta is not None:
            ctx.memo.pop("held", None)         # x changes here: what is held for it no longer describes it
        ctx.ops.add_rmsnorm(x, delta, bias, self.weight, self.eps, out, rows)
        return out


register("norm", "rms", RMSNorm)
