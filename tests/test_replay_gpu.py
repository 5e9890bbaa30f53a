"""-m gpu: the engine's step function (through the trace replay) against the plain implementation, in float32 and
bfloat16: whole prompts; most of a prompt in one step and the last 32 tokens one by one; portions of changing size
down to two tokens; mixed batches of up to four live requests with so few pages that they are used again."""
import numpy as np
import pytest
import torch

from tests import helpers as H

pytestmark = pytest.mark.gpu
CASES = [(n, m) for n in ("A", "B", "C", "D") for m in H.MODES]


def runner_for(tmp, name, mode, max_tokens, options=None):
    from mashbox_b200.engine.replay import make_runner
    dtype, opts = H.MODES[mode]
    folder = H.make_folder(tmp, name, H.store_for(dtype))
    return folder, make_runner(folder, dtype, max_tokens, page_size=H.TINY[name][2], options=dict(opts, **(options or {})))


def replay(runner, steps):
    from mashbox_b200.engine.replay import run_step
    out = {}
    for i, s in enumerate(steps):
        s = dict(s, step=i)
        r = run_step(runner, s)
        if r is not None:
            out[i] = r.numpy()
    return out


@pytest.mark.parametrize("name,mode", CASES)
def test_whole_prompts(tmp_path_factory, name, mode):
    tmp = tmp_path_factory.mktemp("m")
    folder, runner = runner_for(tmp, name, mode, 256)
    for p in H.prompts_for(name, (7, 13, 70, 130)):
        got = replay(runner, [dict(entries=[dict(id="a", tokens=p, want=list(range(len(p))))], end=["a"])])[0]
        H.check(got, folder, p, mode, f"whole prompt of {len(p)}")
    runner.cache.check()


@pytest.mark.parametrize("name,mode", CASES)
def test_last_32_one_by_one(tmp_path_factory, name, mode):
    tmp = tmp_path_factory.mktemp("m")
    folder, runner = runner_for(tmp, name, mode, 192)
    for p in H.prompts_for(name, (40, 150), seed=1):
        cut = len(p) - 32
        steps = [dict(entries=[dict(id="a", tokens=p[:cut], want=[cut - 1])], end=[])]
        steps += [dict(entries=[dict(id="a", tokens=[p[i]], want=[0])], end=["a"] if i == len(p) - 1 else [])
                  for i in range(cut, len(p))]
        out = replay(runner, steps)
        got = np.concatenate([out[i] for i in range(len(steps))])
        H.check(got, folder, p, mode, f"prompt of {len(p)}, last 32 decoded", slice(cut - 1, None))
    runner.cache.check()


@pytest.mark.parametrize("name,mode", CASES)
def test_portions_of_changing_size(tmp_path_factory, name, mode):
    tmp = tmp_path_factory.mktemp("m")
    folder, runner = runner_for(tmp, name, mode, 192)
    p = H.prompts_for(name, (171,), seed=2)[0]
    sizes, at, steps = [2, 17, 3, 64, 2, 31, 16, 8, 5, 2, 21], 0, []
    for s in sizes:
        s = min(s, len(p) - at)
        if s <= 0:
            break
        steps.append(dict(entries=[dict(id="a", tokens=p[at:at + s], want=list(range(s)))], end=[]))
        at += s
    assert at == len(p)
    out = replay(runner, steps)
    got = np.concatenate([out[i] for i in range(len(steps))])
    H.check(got, folder, p, mode, "portions")


def mixed_trace(prompts, rng, max_live=4):
    """Random schedule: up to max_live live requests, each step feeds some of them a portion (2..24 tokens) or, near
    their end, single tokens; a finished request ends and a new one starts on the pages it gave back."""
    todo = list(enumerate(prompts))
    live, steps, where = {}, [], {}
    while todo or live:
        while todo and len(live) < max_live:
            i, p = todo.pop(0)
            live[i] = 0
        entries, end = [], []
        for i in list(live):
            if rng.random() < 0.25 and len(live) > 1:
                continue                                   # left out of this step, goes on later
            p, at = prompts[i], live[i]
            left = len(p) - at
            n = 1 if left <= 6 else int(min(left, rng.integers(2, 25)))
            want = list(range(n))
            entries.append(dict(id=f"r{i}", tokens=p[at:at + n], want=want))
            where.setdefault(i, []).append((len(steps), len([w for e in entries[:-1] for w in e["want"]]), n))
            live[i] += n
            if live[i] == len(p):
                end.append(f"r{i}")
                del live[i]
        if entries:
            steps.append(dict(entries=entries, end=end))
    return steps, where


@pytest.mark.parametrize("name,mode", CASES)
def test_mixed_batches_with_page_reuse(tmp_path_factory, name, mode):
    tmp = tmp_path_factory.mktemp("m")
    lengths = (50, 33, 64, 20, 61, 47, 9, 58)
    prompts = H.prompts_for(name, lengths, seed=3)
    folder, runner = runner_for(tmp, name, mode, 4 * 64)         # four live requests of at most 64 tokens
    steps, where = mixed_trace(prompts, np.random.default_rng(5))
    out = replay(runner, steps)
    for i, p in enumerate(prompts):
        got = np.concatenate([out[s][o:o + n] for s, o, n in where[i]])
        H.check(got, folder, p, mode, f"mixed, request {i}")
    runner.cache.check()
    assert all(f == runner.cache.num_pages for f in runner.cache.free_pages())


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_streaming_products_for_steps_of_few_tokens(tmp_path_factory, name):
    """the weight-streaming products (off by default) take every step of at most 16 tokens: norm, rotation, cache write,
    gate and residual add inside the four products of a layer, the sums of squares handed from one to the next"""
    import mashbox_b200.ops as ops
    tmp = tmp_path_factory.mktemp("m")
    before = dict(ops.STREAM)
    ops.STREAM["tokens"] = 16
    try:
        folder, runner = runner_for(tmp, name, "bf16", 4 * 64)
        p = H.prompts_for(name, (150,), seed=1)[0]
        cut = len(p) - 32
        steps = [dict(entries=[dict(id="a", tokens=p[:cut], want=[cut - 1])], end=[])]
        steps += [dict(entries=[dict(id="a", tokens=[p[i]], want=[0])], end=["a"] if i == len(p) - 1 else [])
                  for i in range(cut, len(p))]
        out = replay(runner, steps)
        H.check(np.concatenate([out[i] for i in range(len(steps))]), folder, p, "bf16", "last 32 decoded", slice(cut - 1, None))
        prompts = H.prompts_for(name, (50, 33, 64, 20, 61, 47, 9, 58), seed=3)
        steps, where = mixed_trace(prompts, np.random.default_rng(5), max_live=2)
        assert sum(1 for s in steps if 2 <= sum(len(e["tokens"]) for e in s["entries"]) <= 16) >= 5
        out = replay(runner, steps)
        for i, q in enumerate(prompts):
            got = np.concatenate([out[s][o:o + n] for s, o, n in where[i]])
            H.check(got, folder, q, "bf16", f"mixed, request {i}")
        runner.cache.check()
    finally:
        ops.STREAM.update(before)


def np_logit_hash(lg):
    """sum over v of bits(lg[v]) * (2 v + 1) mod 2^32 (src/mashbox/runtime/engine.py:80-84) and the top-2 gap, per row"""
    lg = np.ascontiguousarray(lg, np.float32)
    u = lg.view(np.uint32).astype(np.uint64)
    k = (2 * np.arange(lg.shape[1], dtype=np.uint64) + 1)
    h = (u * k % (1 << 32)).sum(-1) % (1 << 32)
    top = np.sort(lg, -1)[:, -2:]
    return [(int(a), float(np.float32(t[1]) - np.float32(t[0]))) for a, t in zip(h, top)]


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_float32_logits_are_bit_identical_under_every_cut(tmp_path_factory, name):
    """What the 32-bit path promises: the logits of a position are the same BITS whether the request ran whole, with its
    last 32 tokens one by one, in portions of changing size down to two tokens, or mixed with other requests on pages
    that were used before.  Every float32 kernel gives each output element one accumulator and a fixed order that does
    not depend on the step (gemm_f32.cu, attention_simple.cu, the norm's fixed tree), so this is equality, not a bar.
    The device-side logit hash must say the same."""
    from mashbox_b200.engine.replay import run_step
    tmp = tmp_path_factory.mktemp("m")
    lengths = (50, 33, 64, 20, 61, 47, 9, 58)
    prompts = H.prompts_for(name, lengths, seed=3)
    folder, runner = runner_for(tmp, name, "f32", 4 * 64)
    whole = [replay(runner, [dict(entries=[dict(id="w", tokens=p, want=list(range(len(p))))], end=["w"])])[0]
             for p in prompts]
    for p, w in zip(prompts, whole):                                     # beside the bar against the plain model
        H.check(w, folder, p, "f32", "whole")
    # last 32 one by one
    for p, w in zip(prompts[:3], whole[:3]):
        cut = max(1, len(p) - 32)
        steps = [dict(entries=[dict(id="a", tokens=p[:cut], want=list(range(cut)))], end=[])]
        steps += [dict(entries=[dict(id="a", tokens=[t], want=[0])], end=[]) for t in p[cut:]]
        steps[-1]["end"] = ["a"]
        out = replay(runner, steps)
        assert np.array_equal(np.concatenate([out[i] for i in range(len(steps))]), w), "last 32 one by one"
    # portions of changing size
    p, w = prompts[2], whole[2]
    at, steps = 0, []
    for s in [2, 17, 3, 2, 31, 9]:
        s = min(s, len(p) - at)
        steps.append(dict(entries=[dict(id="a", tokens=p[at:at + s], want=list(range(s)))], end=[]))
        at += s
    assert at == len(p)
    steps[-1]["end"] = ["a"]
    out = replay(runner, steps)
    assert np.array_equal(np.concatenate([out[i] for i in range(len(steps))]), w), "portions"
    # mixed, up to four live, pages used again; the hash kernel on the same rows
    steps, where = mixed_trace(prompts, np.random.default_rng(5))
    out, hashes = {}, {}
    for i, s in enumerate(steps):
        r = run_step(runner, dict(s, step=i))
        out[i] = r.numpy()
    for i, (p, w) in enumerate(zip(prompts, whole)):
        got = np.concatenate([out[s][o:o + n] for s, o, n in where[i]])
        assert np.array_equal(got, w), f"mixed, request {i}"
    runner.cache.check()
    assert all(f == runner.cache.num_pages for f in runner.cache.free_pages())


def test_trace_run_writes_the_logit_hash(tmp_path):
    """replay with --trace: the device's hash and gap of every wanted row equal numpy's on the logits it wrote"""
    import json

    from mashbox_b200.engine.replay import run_step
    folder, runner = runner_for(tmp_path, "B", "f32", 128)
    p = H.prompts_for("B", (40,), seed=8)[0]
    out = tmp_path / "out"
    out.mkdir()
    lg = run_step(runner, dict(step=3, entries=[dict(id="a", tokens=p, want=[0, 5, 39])], end=["a"]), str(out), trace=True)
    lh = json.load(open(out / "3.lh.json"))
    want = np_logit_hash(lg.numpy())
    assert [(int(h), float(g)) for h, g in lh] == want
    assert np.array_equal(np.fromfile(out / "3.f32", "<f4").reshape(3, -1), lg.numpy())
