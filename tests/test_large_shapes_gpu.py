"""-m gpu: the step function at the layer sizes of an 8B-class model (width 4,096, 32 heads over 8 kv heads of 128,
feed-forward 14,336, vocabulary 128,256; two layers, random weights made on the GPU), where the kernels that tiny
models never select do the work: the tcgen05 attention and gate/up product on prompt portions, the TMA attention with
its splits, the matrix-vector products of small decode batches, captured graphs.

A plain float64 model of this size on the CPU would take minutes, so the references here are the engine's own paths
that the tiny-model tests pin to the plain implementation: the float32 path (NMSE <= 1e-10 there) stands for the exact
logits, and bfloat16 with the plain attention kernel, whole prompt, measures bfloat16's own noise at this size.  The
serving kernels must stay within twice that noise however the tokens are cut into steps, and the float32 path must give
the same logits decoded as whole."""
import numpy as np
import pytest
import torch

from tests.tolerances import BF16_NOISE_FACTOR, assert_logits, nmse

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
CFG = dict(architectures=["LlamaForCausalLM"], hidden_size=4096, intermediate_size=14336, num_attention_heads=32,
           num_key_value_heads=8, num_hidden_layers=2, vocab_size=128256, rms_norm_eps=1e-5, rope_theta=500000.0,
           max_position_embeddings=131072, tie_word_embeddings=False,
           rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                             original_max_position_embeddings=8192))


def make_runner(dtype, max_tokens, options=None):
    from mashbox_b200 import ops
    from mashbox_b200.config.engine import EngineConfig
    from mashbox_b200.config.registry import read_config
    from mashbox_b200.engine.loading import build_model
    from mashbox_b200.engine.runner import ModelRunner
    from mashbox_b200.weights.random_init import RandomSource
    entry, config = read_config(CFG)
    # the same bfloat16 values for every runner; the float32 runner widens them
    source = RandomSource(entry.stored_tensors(config), 7, torch.bfloat16, DEV, std=0.02, norm_std=0.05)
    model = build_model(CFG, source, dtype, DEV, ops=ops)
    cfg = EngineConfig(dtype=dtype, page_size=16, max_tokens=max_tokens, max_requests=4, max_tokens_per_step=1024,
                       chunk=1024, device=DEV)
    return ModelRunner(model, cfg, options)


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


def test_8b_layer_sizes_in_every_cut():
    rng = np.random.default_rng(11)
    a = rng.integers(0, CFG["vocab_size"], 600).tolist()
    b = rng.integers(0, CFG["vocab_size"], 333).tolist()
    wa = [0, 1, 2, 100, 255, 256, 257] + list(range(568, 600))
    wb = [0, 17] + list(range(301, 333))
    decode_sizes = [568] + [1] * 32

    exact = make_runner("float32", 1024)
    ref_a = run(exact, cut_steps("a", a, [600], wa))
    ref_b = run(exact, cut_steps("b", b, [333], wb))
    again = run(exact, cut_steps("a", a, decode_sizes, wa))
    assert_logits(again, ref_a, "float32", "float32, last 32 decoded, against whole")
    del exact
    torch.cuda.empty_cache()

    plain = make_runner("bfloat16", 1024, dict(plain_attention=True, no_graphs=True))
    noise_a = nmse(run(plain, cut_steps("a", a, [600], wa)), ref_a)
    noise_b = nmse(run(plain, cut_steps("b", b, [333], wb)), ref_b)
    del plain
    torch.cuda.empty_cache()
    assert 1e-7 < noise_a < 1e-3 and 1e-7 < noise_b < 1e-3, (noise_a, noise_b)

    def check(got, ref, noise, what):
        assert np.isfinite(got).all(), what
        e = nmse(got, ref)
        assert e <= BF16_NOISE_FACTOR * noise, f"{what}: NMSE {e:.3e}, bfloat16's own noise here {noise:.3e}"
        # the wanted token of the exact model stays the best or within the noise of it
        top = ref.argmax(-1)
        gap = got.max(-1) - got[np.arange(len(top)), top]
        assert (gap <= 0.05 * np.abs(ref).max()).all(), what

    serve = make_runner("bfloat16", 1024)               # 600 -> 640 and 333 -> 384 tokens: the pool is full with both
    check(run(serve, cut_steps("a", a, [600], wa)), ref_a, noise_a, "whole")
    check(run(serve, cut_steps("a", a, decode_sizes, wa)), ref_a, noise_a, "last 32 decoded")
    check(run(serve, cut_steps("a", a, decode_sizes, wa)), ref_a, noise_a, "last 32 decoded, the second time (graphs)")
    check(run(serve, cut_steps("a", a, [2, 254, 3, 129, 2, 178, 32], wa)), ref_a, noise_a, "portions")
    # mixed: portions of a beside portions of b, then 32 steps with a decoded token of each (on pages used before)
    sa, sb = cut_steps("a", a, [300, 268] + [1] * 32, wa), cut_steps("b", b, [2, 299] + [1] * 32, wb)
    steps, got_a, got_b = [], [], []
    for i in range(max(len(sa), len(sb))):
        entries, end = [], []
        for s in ([sa[i]] if i < len(sa) else []) + ([sb[i]] if i < len(sb) else []):
            entries += s["entries"]
            end += s["end"]
        steps.append(dict(entries=entries, end=end))
    from mashbox_b200.engine.replay import run_step
    for i, s in enumerate(steps):
        r = run_step(serve, dict(s, step=i))
        if r is None:
            continue
        r, o = r.cpu().numpy(), 0
        for e in s["entries"]:
            n = len(e["want"])
            (got_a if e["id"] == "a" else got_b).append(r[o:o + n])
            o += n
    check(np.concatenate(got_a), ref_a, noise_a, "mixed, request a")
    check(np.concatenate(got_b), ref_b, noise_b, "mixed, request b")
    serve.cache.check()
    assert serve.cache.free_pages() == [serve.cache.num_pages]
    assert serve.stats["graph_replays"] > 0
