"""Dense SwiGLU feed-forward: (silu(h Wg^T) * (h Wu^T)) Wd^T, silu and the product in float32
(src/mashbox/gguf/archs/dense.py:356-357).  Gate and up weights are concatenated at load so one product makes both."""
from ..weights.loader import Want
from .base import register


class SwiGLU:
    graph_safe = True       # forward() depends on the batch only through the lengths of the step's arrays
    def __init__(self, hidden, intermediate, prefix="", names=None):
        self.D, self.F = int(hidden), int(intermediate)
        n = dict(gate="ffn_gate", up="ffn_up", down="ffn_down")
        n.update(names or {})
        self.names = {k: prefix + v + ".weight" for k, v in n.items()}
        self.wgu = self.wd = None

    def wants(self):
        return [Want(self.names["gate"], (self.F, self.D), "matrix"), Want(self.names["up"], (self.F, self.D), "matrix"),
                Want(self.names["down"], (self.D, self.F), "matrix")]

    def bind(self, tensors, env):
        import torch
        self.wgu = torch.cat([tensors[self.names["gate"]], tensors[self.names["up"]]], 0).contiguous()
        self.wd = tensors[self.names["down"]]

    fuses_small = True      # forward() takes normed= and residual= (see PreNormBlock)

    def forward(self, ctx, h, normed=None, residual=None):
        import torch
        N = ctx.N
        a = ctx.ws.get("ffn_act", N, (self.F,), ctx.dtype)
        if normed is not None:
            x, norm = normed
            w, eps = norm.fusable()
            ctx.ops.linear_small_normed(x, w, eps, self.wgu, a, "swiglu", held=ctx.take_held(x, norm))
        elif ctx.dtype == torch.bfloat16 and ctx.ops.fused_swiglu_supports(N, self.F, self.D):
            ctx.ops.linear_swiglu(h, self.wgu, a)           # both products and the gate in one kernel
        else:
            gu = ctx.ws.get("gate_up", N, (2 * self.F,), ctx.dtype)
            ctx.ops.linear(h, self.wgu, out=gu)
            ctx.ops.swiglu(gu, a)
        if residual is not None:
            ctx.add_into_stream(a, self.wd, residual)
            return None
        y = ctx.ws.get("delta", N, (self.D,), ctx.dtype)
        ctx.ops.linear(a, self.wd, out=y)
        return y, None


register("feed_forward", "swiglu", SwiGLU)
