"""Block arrangements: how a layer's norm, mixer and feed-forward are put together.

"prenorm": x += mixer(norm1(x)); x += ffn(norm2(x)) (src/mashbox/gguf/archs/dense.py:339-357).  The adds are deferred: a
sublayer returns its output as `pending` and the next norm adds it into the float32 residual stream in the same kernel
that normalises, so the block returns the feed-forward's output still pending.
"""
from .base import make, register


class PreNormBlock:
    graph_safe = True       # forward() depends on the batch only through the lengths of the step's arrays
    def __init__(self, prefix, mixer, ffn, norm=None, norm1=None, norm2=None):
        """mixer, ffn: part specs; norm: the spec of both norms, or norm1 / norm2 when they differ"""
        p = prefix
        self.norm1 = make("norm", norm1 or norm, name=p + "attn_norm.weight")
        self.mixer = make("mixer", mixer, prefix=p)
        self.norm2 = make("norm", norm2 or norm, name=p + "ffn_norm.weight")
        self.ffn = make("feed_forward", ffn, prefix=p)

    def parts(self):
        return [self.norm1, self.mixer, self.norm2, self.ffn]

    def forward(self, ctx, x, pending, run):
        # A step of very few tokens is a chain of short kernels.  Parts that say `fuses_small` take two of them in:
        # with normed=(x, norm) their first product is the product of the normalised stream without a norm kernel (x
        # must be up to date: nothing pending; the streaming products also need what the product before left for this
        # norm, ctx.held_for), with residual=x their last product adds into the stream (ctx.add_into_stream) and
        # nothing is left pending.
        small = ctx.ops.small_fused_supports(ctx.N, x.shape[1], ctx.dtype) and not ctx.options.get("no_small_fusion", False)
        pending = self._sublayer(ctx, x, pending, self.norm1, self.mixer, small, self.norm2, run)
        return self._sublayer(ctx, x, pending, self.norm2, self.ffn, small, ctx.next_first_norm)

    def first_norm(self):
        """the norm that reads the residual stream first when this block runs"""
        return self.norm1

    @staticmethod
    def _sublayer(ctx, x, pending, norm, part, small, after, *run):
        ctx.after_norm = after                  # the norm that reads x after this part (None: not known)
        if not (small and getattr(part, "fuses_small", False) and hasattr(norm, "fusable")):
            return part.forward(ctx, norm.forward(ctx, x, pending), *run)
        ready = pending is None and (not ctx.ops.small_normed_needs_held(ctx.N, x.shape[1]) or ctx.held_for(x, norm) is not None)
        if not ready:
            return part.forward(ctx, norm.forward(ctx, x, pending), *run, residual=x)
        return part.forward(ctx, None, *run, normed=(x, norm), residual=x)


register("block", "prenorm", PreNormBlock)
