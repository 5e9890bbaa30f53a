"""-m gpu: programmatic dependent launch (engine option "pdl") changes WHEN the kernels of a small step start, never
what they compute: with it a kernel may be resident while the one before it still runs, and waits for it by itself
before it reads what that kernel wrote.  The logits of every step must be the same bits with the option on and off --
steps of one token (the matrix-vector kernels), of 2 to 16 tokens (the weight-streaming products), decode batches
beside prompt portions, replayed from captured graphs -- and equal to the plain implementation within the usual bar."""
import numpy as np
import pytest
import torch

from tests import helpers as H
from tests.test_replay_gpu import mixed_trace, replay, runner_for

pytestmark = pytest.mark.gpu


def steps_for(name):
    prompts = H.prompts_for(name, (150, 47, 90), seed=21)
    steps = []
    # request a: most of the prompt, then 40 single tokens (twice the same shapes: the second time from graphs)
    p = prompts[0]
    cut = len(p) - 40
    steps.append(dict(entries=[dict(id="a", tokens=p[:cut], want=[cut - 1])], end=[]))
    steps += [dict(entries=[dict(id="a", tokens=[t], want=[0])], end=[]) for t in p[cut:]]
    # b and c join: portions of 2 to 7 tokens of each beside a's ... no more tokens of a; then decode batches of 2
    b, c = prompts[1], prompts[2]
    steps.append(dict(entries=[dict(id="b", tokens=b[:40], want=[39]), dict(id="c", tokens=c[:5], want=[4])], end=["a"]))
    at_b, at_c = 40, 5
    while at_b < len(b) or at_c < len(c):
        entries = []
        if at_b < len(b):
            entries.append(dict(id="b", tokens=[b[at_b]], want=[0]))
            at_b += 1
        if at_c < len(c):
            n = min(7, len(c) - at_c)
            entries.append(dict(id="c", tokens=c[at_c:at_c + n], want=list(range(n))))
            at_c += n
        steps.append(dict(entries=entries, end=[]))
    steps[-1]["end"] = ["b", "c"]
    return prompts, steps


@pytest.mark.parametrize("name", ["C", "D", "B"])
def test_pdl_changes_no_bit(tmp_path_factory, name):
    import mashbox_b200.ops as ops
    tmp = tmp_path_factory.mktemp("m")
    prompts, steps = steps_for(name)
    try:
        # the same kernels with and without the launch attribute (by itself "pdl": False also hands one-token steps
        # back to the matrix-vector kernels: that combination is checked against the plain model below)
        folder, off = runner_for(tmp, name, "bf16", 512, options={"pdl": False, "gemv_tokens": 0})
        want = replay(off, steps)
        want2 = replay(off, steps)                     # the second pass replays captured graphs
        del off
        folder, on = runner_for(tmp, name, "bf16", 512, options={"pdl": True, "gemv_tokens": 0})
        assert ops.PDL["on"]
        got = replay(on, steps)
        got2 = replay(on, steps)
        assert on.stats["graph_replays"] > 0
        del on
        folder, plainly = runner_for(tmp, name, "bf16", 512, options={"pdl": False})
        assert ops.GEMV["fused"] == 1 and not ops.PDL["on"]
        gemv = replay(plainly, steps)
    finally:
        ops.configure({})
    for i in want:
        assert np.array_equal(want[i], want2[i])
        assert np.array_equal(got[i], want[i]), f"step {i}: logits differ with programmatic dependent launch on"
        assert np.array_equal(got2[i], want[i]), f"step {i}, from a graph: logits differ"
    # and the usual bar against the plain implementation, for request a's decoded tokens
    p = prompts[0]
    cut = len(p) - 40
    H.check(np.concatenate([got[i] for i in range(41)]), folder, p, "bf16", "request a, decoded", slice(cut - 1, None))
    H.check(np.concatenate([gemv[i] for i in range(41)]), folder, p, "bf16", "request a, decoded by the matrix-vector kernels",
            slice(cut - 1, None))


def test_pdl_under_random_mixed_traffic(tmp_path_factory):
    """up to four live requests, portions of some beside decoded tokens of others, pages used again: the same bits"""
    import mashbox_b200.ops as ops
    tmp = tmp_path_factory.mktemp("m")
    prompts = H.prompts_for("C", (50, 33, 64, 20, 61, 47, 9, 58), seed=3)
    steps, where = mixed_trace(prompts, np.random.default_rng(7))
    try:
        _, off = runner_for(tmp, "C", "bf16", 4 * 64, options={"pdl": False, "gemv_tokens": 0})
        want = replay(off, steps)
        del off
        _, on = runner_for(tmp, "C", "bf16", 4 * 64, options={"pdl": True, "gemv_tokens": 0})
        got = replay(on, steps)
    finally:
        ops.configure({})
    assert all(np.array_equal(got[i], want[i]) for i in want)
