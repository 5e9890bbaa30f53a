"""Block arrangements: how a layer's norm, mixer and feed-forward are put together.

"prenorm": x += mixer(norm1(x)); x += ffn(norm2(x)) (src/mashbox/gguf/archs/dense.py:339-357).  The adds are deferred: a
sublayer returns its output as `pending` and the next norm adds it into the float32 residual stream in the same kernel
that normalises, so the block returns the feed-forward's output still pending.
"""
from .base import make, register


class PreNormBlock:
    graph_safe = True       # forward() depends on the batch only through the lengths of the step's arrays
    def __init__(self, layer):
        p = layer.prefix
        self.norm1 = make("norm", layer.norm, name=p + "attn_norm.weight")
        self.mixer = make("mixer", layer.mixer, prefix=p)
        self.norm2 = make("norm", layer.norm, name=p + "ffn_norm.weight")
        self.ffn = make("feed_forward", layer.ffn, prefix=p)

    def parts(self):
        return [self.norm1, self.mixer, self.norm2, self.ffn]

    def forward(self, ctx, x, pending, run):
        h = self.norm1.forward(ctx, x, pending)
        y = self.mixer.forward(ctx, h, run)
        h = self.norm2.forward(ctx, x, y)
        return self.ffn.forward(ctx, h)


register("block", "prenorm", PreNormBlock)
