"""-m "not gpu": what PreNormBlock asks of its parts on steps of few tokens, with scripted ops on the CPU: which
sublayers get `normed=` and `residual=`, and that what a product leaves for the norm after it is handed on only to that
norm, only for the same stream, and only once."""
import types

import torch

from mashbox_b200.parts.base import StepContext, Workspace
from mashbox_b200.parts.block import PreNormBlock


class Norm:
    def __init__(self, log, name):
        self.log, self.name, self.w = log, name, torch.ones(64)

    def fusable(self):
        return self.w, 1e-5

    def forward(self, ctx, x, pending=None, rows=None):
        if pending is not None:
            ctx.memo.pop("held", None)
        self.log.append(("norm kernel", self.name, pending is not None))
        return "normed by " + self.name


class Part:
    fuses_small = True

    def __init__(self, log, name):
        self.log, self.name = log, name

    def forward(self, ctx, h, *run, normed=None, residual=None):
        held = None
        if normed is not None:
            x, norm = normed
            held = ctx.take_held(x, norm)
        self.log.append((self.name, h, normed is not None, held is not None, residual is not None))
        if residual is not None:
            ctx.add_into_stream("a", "w", residual)
            return None
        return "delta of " + self.name, None


class Ops:
    def __init__(self, needs_held, fills):
        self.needs_held, self.fills, self.calls = needs_held, fills, []

    def small_fused_supports(self, N, K, dtype):
        return True

    def small_normed_needs_held(self, N, K):
        return self.needs_held

    def linear_small_residual(self, a, w, x, bias=None, sums=None, next_w=None, scaled=None):
        self.calls.append((sums is not None, next_w is not None, scaled is not None))
        return self.fills and sums is not None and scaled is not None


def make(needs_held=True, fills=True):
    log = []
    ops = Ops(needs_held, fills)
    env = types.SimpleNamespace(ops=ops, dtype=torch.bfloat16, device="cpu")
    ctx = StepContext(env, None, Workspace("cpu", 8), None, None, {})
    ctx.N = 4
    block = PreNormBlock.__new__(PreNormBlock)
    block.norm1, block.norm2 = Norm(log, "norm1"), Norm(log, "norm2")
    block.mixer, block.ffn = Part(log, "mixer"), Part(log, "ffn")
    return log, ops, ctx, block


def test_first_sublayer_runs_its_norm_then_everything_is_handed_on():
    log, ops, ctx, block = make()
    x = torch.zeros(4, 64)
    nxt = Norm(log, "next block's norm1")
    ctx.next_first_norm = nxt
    assert block.forward(ctx, x, None, "run") is None
    assert log == [("norm kernel", "norm1", False), ("mixer", "normed by norm1", False, False, True),
                   ("ffn", None, True, True, True)]
    assert ops.calls == [(True, True, True), (True, True, True)]
    assert ctx.held_for(x, nxt) is not None and ctx.held_for(x, block.norm1) is None
    assert ctx.held_for(torch.zeros(4, 64), nxt) is None            # another stream
    assert ctx.take_held(x, nxt) is not None and ctx.take_held(x, nxt) is None     # used up


def test_nothing_to_hand_on_when_the_next_norm_is_unknown_or_the_kernel_does_not_fill():
    log, ops, ctx, block = make()
    x = torch.zeros(4, 64)
    ctx.next_first_norm = None
    block.forward(ctx, x, None, "run")
    assert ops.calls[-1] == (False, False, False) and ctx.memo.get("held") is None
    log2, ops2, ctx2, block2 = make(fills=False)                    # e.g. the matrix-vector kernels
    ctx2.next_first_norm = Norm(log2, "n")
    block2.forward(ctx2, x, None, "run")
    assert ctx2.memo.get("held") is None
    assert log2[2] == ("norm kernel", "norm2", False) and log2[3] == ("ffn", "normed by norm2", False, False, True)


def test_kernels_that_normalise_by_themselves_need_nothing_held():
    log, ops, ctx, block = make(needs_held=False, fills=False)
    x = torch.zeros(4, 64)
    block.forward(ctx, x, None, "run")
    assert log == [("mixer", None, True, False, True), ("ffn", None, True, False, True)]


def test_a_pending_delta_goes_through_the_norm_kernel_and_drops_what_was_held():
    log, ops, ctx, block = make()
    x = torch.zeros(4, 64)
    ctx.memo["held"] = (x.data_ptr(), block.norm1, "sums", "scaled")
    block.forward(ctx, x, ("delta", None), "run")
    assert log[0] == ("norm kernel", "norm1", True)
    assert log[1] == ("mixer", "normed by norm1", False, False, True)


def test_signature_of_step_inputs_ends_at_the_mark():
    """arrays added after mark() (the sampler's settings) are sent with the step but are not part of a graph's shape"""
    from mashbox_b200.parts.base import StepInputs
    inp = StepInputs(None)
    inp.add("a", [1, 2, 3])
    inp.add("b", [])
    assert inp.signature() == (("a", 3), ("b", 0))
    inp.mark()
    inp.add("sample_rows", [0] * 7)
    assert inp.signature() == (("a", 3), ("b", 0)) and inp.has("sample_rows")
    inp.reset()
    inp.add("a", [1])
    inp.add("late", [2, 3])
    assert inp.signature() == (("a", 1), ("late", 2))
