"""-m gpu: the step function at the layer sizes of an 8B-class model (width 4,096, 32 heads over 8 kv heads of 128,
feed-forward 14,336, vocabulary 128,256; two layers, random weights made on the GPU), where the kernels that tiny
models never select do the work: the tcgen05 attention and gate/up product on prompt portions, the TMA attention with
its splits, the matrix-vector and weight-streaming products of small decode batches, the library path of decode
batches of 17 to 127 tokens, captured graphs.

The reference is the PLAIN implementation (tests/plain/llama.py: whole sequences, no cache, float64), run on the GPU
because a float64 model of this size takes minutes on the CPU; its head runs on the wanted rows only.  It shares no
code with the package.  float32 engine: NMSE against it under the bar for this size (tests/tolerances.py), and the same
BITS decoded as whole.  bfloat16 engine: within twice bfloat16's own noise, which is the plain model with bfloat16
storage against the exact one, however the tokens are cut into steps."""
import numpy as np
import pytest
import torch

from tests.plain import llama as plain
from tests.tolerances import BF16_NOISE_FACTOR, NMSE_F32_LARGE, nmse

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
CFG = dict(architectures=["LlamaForCausalLM"], hidden_size=4096, intermediate_size=14336, num_attention_heads=32,
           num_key_value_heads=8, num_hidden_layers=2, vocab_size=128256, rms_norm_eps=1e-5, rope_theta=500000.0,
           max_position_embeddings=131072, tie_word_embeddings=False,
           rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                             original_max_position_embeddings=8192))


def weights():
    from mashbox_b200.config.registry import read_config
    from mashbox_b200.weights.random_init import RandomSource
    entry, config = read_config(CFG)
    # the same bfloat16 values for every runner and for the plain model; the float32 runner widens them
    return RandomSource(entry.stored_tensors(config), 7, torch.bfloat16, DEV, std=0.02, norm_std=0.05)


def make_runner(dtype, max_tokens, options=None, max_requests=4):
    from mashbox_b200 import ops
    from mashbox_b200.config.engine import EngineConfig
    from mashbox_b200.engine.loading import build_model
    from mashbox_b200.engine.runner import ModelRunner
    model = build_model(CFG, weights(), dtype, DEV, ops=ops)
    cfg = EngineConfig(dtype=dtype, page_size=16, max_tokens=max_tokens, max_requests=max_requests,
                       max_tokens_per_step=1024, chunk=1024, device=DEV)
    return ModelRunner(model, cfg, options)


class PlainOnGpu:
    """the plain model with its float64 tensors on the GPU: exact logits and logits with bfloat16 storage, at the
    wanted rows of a whole sequence"""

    def __init__(self):
        src = weights()
        self.W = {n: src.get(n).to(torch.float64) for n in src.names()}

    def exact(self, tokens, rows):
        return plain.forward(CFG, self.W, tokens, device=DEV, rows=rows).cpu().numpy()

    def rounded(self, tokens, rows):
        return plain.forward(CFG, self.W, tokens, held=plain.round_bf16, device=DEV, rows=rows).cpu().numpy()


def run(runner, steps):
    from mashbox_b200.engine.replay import run_step
    out = []
    for i, s in enumerate(steps):
        r = run_step(runner, dict(s, step=i))
        if r is not None:
            out.append(r.cpu().numpy())
    return np.concatenate(out)


def cut_steps(rid, tokens, sizes, wanted, end=True):
    """the request in portions of the given sizes; the logits of the positions in `wanted` are asked for"""
    steps, at = [], 0
    for n in sizes:
        want = [p - at for p in wanted if at <= p < at + n]
        steps.append(dict(entries=[dict(id=rid, tokens=tokens[at:at + n], want=want)], end=[]))
        at += n
    assert at == len(tokens)
    if end:
        steps[-1]["end"] = [rid]
    return steps


def interleave(runner, plans):
    """plans: {rid: steps of one request}; step i of every request runs as one batch.  -> {rid: logits}"""
    from mashbox_b200.engine.replay import run_step
    got = {r: [] for r in plans}
    for i in range(max(len(s) for s in plans.values())):
        entries, end = [], []
        for r, steps in plans.items():
            if i < len(steps):
                entries += steps[i]["entries"]
                end += steps[i]["end"]
        out = run_step(runner, dict(step=i, entries=entries, end=end))
        if out is None:
            continue
        out, o = out.cpu().numpy(), 0
        for e in entries:
            n = len(e["want"])
            got[e["id"]].append(out[o:o + n])
            o += n
    return {r: np.concatenate(v) for r, v in got.items()}


def test_8b_layer_sizes_in_every_cut():
    rng = np.random.default_rng(11)
    V = CFG["vocab_size"]
    a, b = rng.integers(0, V, 600).tolist(), rng.integers(0, V, 333).tolist()
    c, d = rng.integers(0, V, 150).tolist(), rng.integers(0, V, 270).tolist()
    wa = [0, 1, 2, 100, 255, 256, 257] + list(range(568, 600))
    wb = [0, 17] + list(range(301, 333))
    wc = [5] + list(range(118, 150))
    wd = [31, 32] + list(range(238, 270))
    toks, wants = dict(a=a, b=b, c=c, d=d), dict(a=wa, b=wb, c=wc, d=wd)
    decode_sizes = [568] + [1] * 32

    oracle = PlainOnGpu()
    ref = {r: oracle.exact(toks[r], wants[r]) for r in toks}
    noise = {r: nmse(oracle.rounded(toks[r], wants[r]), ref[r]) for r in toks}
    # a decode batch of 20 requests (the library's products, between the streaming kernels and the tcgen05 ones)
    many = [rng.integers(0, V, int(n)).tolist() for n in rng.integers(40, 90, 20)]
    ref_many = [oracle.exact(t, range(len(t) - 5, len(t))) for t in many]
    noise_many = nmse(np.concatenate([oracle.rounded(t, range(len(t) - 5, len(t))) for t in many]), np.concatenate(ref_many))
    del oracle
    torch.cuda.empty_cache()
    assert all(1e-7 < n < 1e-3 for n in noise.values()), noise

    exact = make_runner("float32", 1024)
    whole = run(exact, cut_steps("a", a, [600], wa))
    e = nmse(whole, ref["a"])
    worst = float(np.abs(whole - ref["a"]).max() / np.abs(ref["a"]).max())
    assert e <= NMSE_F32_LARGE and worst <= 1e-4, f"float32 against the plain model: NMSE {e:.3e}, worst {worst:.3e}"
    assert np.array_equal(run(exact, cut_steps("a", a, decode_sizes, wa)), whole), "float32: decoded and whole differ in bits"
    assert np.array_equal(run(exact, cut_steps("a", a, [2, 254, 3, 129, 2, 178, 32], wa)), whole), "float32: portions"
    del exact
    torch.cuda.empty_cache()

    def check(got, r, what, bar=None, want=None):
        want = ref[r] if want is None else want
        bar = noise[r] if bar is None else bar
        assert got.shape == want.shape and np.isfinite(got).all(), what
        e = nmse(got, want)
        assert e <= BF16_NOISE_FACTOR * bar, f"{what}: NMSE {e:.3e}, bfloat16's own noise here {bar:.3e}"
        # the exact model's best token stays the best or within the noise of it
        top = want.argmax(-1)
        gap = got.max(-1) - got[np.arange(len(top)), top]
        assert (gap <= 0.05 * np.abs(want).max()).all(), what

    serve = make_runner("bfloat16", 1024)               # 600 -> 640 and 333 -> 384 tokens: the pool is full with both
    check(run(serve, cut_steps("a", a, [600], wa)), "a", "whole")
    check(run(serve, cut_steps("a", a, decode_sizes, wa)), "a", "last 32 decoded")
    check(run(serve, cut_steps("a", a, decode_sizes, wa)), "a", "last 32 decoded, the second time (graphs)")
    check(run(serve, cut_steps("a", a, [2, 254, 3, 129, 2, 178, 32], wa)), "a", "portions")
    # two requests mixed: portions of a beside portions of b, then 32 steps with a decoded token of each
    got = interleave(serve, dict(a=cut_steps("a", a, [300, 268] + [1] * 32, wa),
                                 b=cut_steps("b", b, [2, 299] + [1] * 32, wb)))
    check(got["a"], "a", "two mixed, request a")
    check(got["b"], "b", "two mixed, request b")
    serve.cache.check()
    assert serve.cache.free_pages() == [serve.cache.num_pages]
    assert serve.stats["graph_replays"] > 0
    del serve
    torch.cuda.empty_cache()

    # three live requests fill the pool (150 -> 160, 270 -> 272, 333 -> 336 tokens), portions of some beside decoded
    # tokens of others; c ends first and a fourth request (c's tokens again, as "e") runs on the pages it gave back
    four = make_runner("bfloat16", 160 + 272 + 336)
    plans = dict(c=cut_steps("c", c, [118] + [1] * 32, wc),
                 d=cut_steps("d", d, [17, 100, 2, 119] + [1] * 32, wd),
                 b=cut_steps("b", b, [150, 3, 148] + [1] * 32, wb))
    e_steps = cut_steps("e", c, [60, 58] + [1] * 32, wc)
    plans["e"] = [dict(entries=[], end=[])] * 33 + e_steps          # starts when c has ended (33 steps)
    got = interleave(four, plans)
    for r, name in (("c", "c"), ("d", "d"), ("b", "b"), ("e", "c")):
        check(got[r], name, f"four live, request {r}")
    four.cache.check()
    assert four.cache.free_pages() == [four.cache.num_pages]
    del four
    torch.cuda.empty_cache()

    # a decode batch of 20: every request's prompt but its last 5 tokens in steps of four requests, then 5 steps that
    # bring one token of each of the 20
    wide = make_runner("bfloat16", 20 * 96, max_requests=20)
    for i in range(0, 20, 4):
        entries = [dict(id=f"m{j}", tokens=many[j][:-5], want=[]) for j in range(i, i + 4)]
        assert run_none(wide, entries)
    outs = []
    for k in range(5):
        entries = [dict(id=f"m{j}", tokens=[many[j][len(many[j]) - 5 + k]], want=[0]) for j in range(20)]
        from mashbox_b200.engine.replay import run_step
        outs.append(run_step(wide, dict(step=k, entries=entries, end=[f"m{j}" for j in range(20)] if k == 4 else []))
                    .cpu().numpy())
    got_many = np.concatenate([np.stack([o[j] for o in outs]) for j in range(20)])
    check(got_many, None, "decode batch of 20", bar=noise_many, want=np.concatenate(ref_many))
    wide.cache.check()
    assert wide.stats["graph_replays"] > 0                           # the batch of 20 came five times


def run_none(runner, entries):
    from mashbox_b200.engine.replay import run_step
    return run_step(runner, dict(step=0, entries=entries, end=[])) is None
