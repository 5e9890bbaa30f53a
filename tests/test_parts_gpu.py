"""-m gpu: each part of a layer alone against its plain reference, at sizes of its own; the schedule as data (a layer
run twice, a layer that reads another layer's cache); and a toy architecture defined in this file -- a mixer with state
of its own beside an attention layer -- registered, built from a model folder and stepped in several cuts without any
change to the framework's files."""
import json
import os
from dataclasses import dataclass

import numpy as np
import pytest
import torch

from tests import helpers as H
from tests.plain import llama as plain
from tests.tolerances import KERNEL_BF16, KERNEL_F32, assert_logits

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


class PartModel:
    """the least a ModelRunner needs around one mixer (or none)"""
    vocab = 1

    def __init__(self, mixer=None, caches=(0,)):
        self.mixer, self.caches = mixer, caches

    def cache_needs(self):
        if self.mixer is None:
            return {}, {}
        st = self.mixer.state_need()
        return {c: self.mixer.cache_need() for c in self.caches}, ({c: st for c in self.caches} if st else {})

    def prepare(self, ctx):
        if self.mixer is not None:
            self.mixer.prepare(ctx)


def rig(mixer, dtype, page=8, tokens=512, options=None):
    from mashbox_b200.config.engine import EngineConfig
    from mashbox_b200.engine.runner import ModelRunner
    cfg = EngineConfig(dtype=dtype, page_size=page, max_tokens=tokens, max_requests=4, max_tokens_per_step=tokens,
                       chunk=tokens)
    return ModelRunner(PartModel(mixer), cfg, options)


def close(got, want, dtype, what):
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    tol = (KERNEL_F32 if dtype == "float32" else KERNEL_BF16) * float(want.abs().max())
    err = float((got - want).abs().max())
    assert torch.isfinite(got).all() and err <= tol, f"{what}: max error {err:.3e}, bar {tol:.3e}"


def env_for(dtype):
    import mashbox_b200.ops as K
    from mashbox_b200.parts import Env
    return Env(getattr(torch, dtype), torch.device(DEV), K)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_feed_forward_embedding_and_head_alone(dtype):
    from mashbox_b200.parts import PartSpec, make
    g = torch.Generator().manual_seed(0)
    D, F, V, N = 72, 200, 301, 11
    td = getattr(torch, dtype)
    runner = rig(None, dtype)
    runner.cache.admit("a")
    ctx = runner.begin([("a", list(range(N)), [1, 7])])
    env = env_for(dtype)
    # norm
    norm = make("norm", PartSpec("rms", width=D, eps=1e-3), name="n.weight")
    w = 1 + 0.2 * torch.randn(D, generator=g)
    norm.bind({"n.weight": w.to(DEV)}, env)
    x0 = torch.randn(N, D, generator=g)
    delta = torch.randn(N, D, generator=g).to(td)
    x = x0.to(DEV).clone()
    h = norm.forward(ctx, x, (delta.to(DEV), None))
    v = x0.double() + delta.double()
    close(h, plain.rms_norm(v, w.double(), 1e-3), dtype, "norm part")
    close(x, v, "float32", "stream")
    hr = norm.forward(ctx, x, None, rows=ctx.dev("want"))
    close(hr, plain.rms_norm(v, w.double(), 1e-3)[[1, 7]], dtype, "norm part, picked rows")
    # feed-forward
    ffn = make("feed_forward", PartSpec("swiglu", hidden=D, intermediate=F), prefix="l.")
    ws = {n: (torch.randn(s, generator=g) / s[1] ** 0.5).to(td) for n, s in
          (("l.ffn_gate.weight", (F, D)), ("l.ffn_up.weight", (F, D)), ("l.ffn_down.weight", (D, F)))}
    assert {w_.name for w_ in ffn.wants()} == set(ws)
    ffn.bind({k: t.to(DEV) for k, t in ws.items()}, env)
    hin = torch.randn(N, D, generator=g).to(td)
    y, bias = ffn.forward(ctx, hin.to(DEV))
    want = plain.swiglu(hin.double(), ws["l.ffn_gate.weight"].double(), ws["l.ffn_up.weight"].double(),
                        ws["l.ffn_down.weight"].double())
    close(y, want, dtype, "feed-forward part")
    assert bias is None
    # embedding and head (tied)
    emb = make("embedding", PartSpec("table", vocab=V, hidden=D))
    head = make("head", PartSpec("linear", vocab=V, hidden=D, tied=True))
    table = torch.randn(V, D, generator=g).to(td)
    emb.bind({"token_embd.weight": table.to(DEV)}, env)
    head.bind({"token_embd.weight": table.to(DEV)}, env)
    assert head.wants() == []
    xe = torch.empty(N, D, device=DEV)
    emb.forward(ctx, xe)
    assert torch.equal(xe.cpu(), table.float()[:N])
    lg = head.forward(ctx, hin.to(DEV)[:3].contiguous())
    assert lg.dtype == torch.float32
    close(lg, hin[:3].double() @ table.double().T, "float32" if dtype == "float32" else "bfloat16", "head part")


@pytest.mark.parametrize("dtype,options", [("float32", {}), ("bfloat16", {}), ("bfloat16", {"plain_attention": True}),
                                           ("bfloat16", {"attention_target_blocks": 100000})])
@pytest.mark.parametrize("HD,H,KV,window,bias,pairing", [(32, 6, 2, None, True, "adjacent"), (64, 4, 4, 23, False, "halves"),
                                                         (48, 3, 1, None, False, "adjacent"),
                                                         (256, 2, 1, 40, False, "halves")])
def test_attention_mixer_alone_in_three_cuts(dtype, options, HD, H, KV, window, bias, pairing):
    """the mixer over its own paged cache: a whole sequence at once, in portions, and token by token beside another
    sequence, against the plain functions (projections, rotation, attention) over the whole sequence"""
    from mashbox_b200.parts import LayerRun, PartSpec, make
    g = torch.Generator().manual_seed(1)
    D, T = 80, 75
    td = getattr(torch, dtype)
    rope = PartSpec("rope", head_dim=HD, rotary_dim=HD // 2, theta=10000.0, scaling=("linear", 2.0), pairing=pairing)
    mixer = make("mixer", PartSpec("attention", hidden=D, heads=H, kv_heads=KV, head_dim=HD, bias=bias, position=rope,
                                   window=window), prefix="b.")
    shapes = {w.name: w.shape for w in mixer.wants()}
    ws = {n: ((torch.randn(s, generator=g) / s[-1] ** 0.5) if len(s) == 2 else 0.3 * torch.randn(s, generator=g))
          for n, s in shapes.items()}
    ws = {n: (t.to(td) if t.ndim == 2 else t) for n, t in ws.items()}
    mixer.bind({n: t.to(DEV) for n, t in ws.items()}, env_for(dtype))
    runner = rig(mixer, dtype, page=8, options=options)
    hs = {r: torch.randn(T, D, generator=g).to(td) for r in ("a", "b")}

    def reference(h):
        f = lambda n: ws[n].double()
        b = lambda n: f(n) if bias else None
        hh = h.double()
        q = plain.linear(hh, f("b.attn_q.weight"), b("b.attn_q.bias")).reshape(T, H, HD)
        k = plain.linear(hh, f("b.attn_k.weight"), b("b.attn_k.bias")).reshape(T, KV, HD)
        v = plain.linear(hh, f("b.attn_v.weight"), b("b.attn_v.bias")).reshape(T, KV, HD)
        fr = plain.rope_frequencies(10000.0, HD // 2, dict(rope_type="linear", factor=2.0))
        rot = plain.rope_adjacent if pairing == "adjacent" else plain.rope_halves
        q, k = rot(q, np.arange(T), fr), rot(k, np.arange(T), fr)
        o = plain.attention(q, k, v, HD ** -0.5, window=window)
        return plain.linear(o, f("b.attn_output.weight"), b("b.attn_output.bias"))

    def step(entries):
        ctx = runner.begin([(r, [0] * n, []) for r, _, n in entries])
        hin = torch.cat([hs[r][at:at + n] for r, at, n in entries]).to(DEV)
        y, bo = mixer.forward(ctx, hin, LayerRun(layer=0, cache=0, write=True))
        y = y.float() + (bo if bo is not None else 0.0)
        runner.commit([(r, [0] * n, []) for r, _, n in entries])
        runner.check()
        return y.cpu()

    want = {r: reference(hs[r]) for r in hs}
    runner.cache.admit("a")
    close(step([("a", 0, T)]), want["a"], dtype, "whole")
    runner.cache.release("a")
    runner.cache.admit("a")
    got = torch.cat([step([("a", at, n)]) for at, n in ((0, 2), (2, 31), (33, 9), (42, 33))])
    close(got, want["a"], dtype, "portions")
    runner.cache.release("a")
    runner.cache.admit("a")
    runner.cache.admit("b")
    outs = {"a": [], "b": []}
    y = step([("a", 0, 40), ("b", 0, 3)])
    outs["a"].append(y[:40]); outs["b"].append(y[40:])
    for i in range(35):
        y = step([("a", 40 + i, 1), ("b", 3 + 2 * i, 2)])
        outs["a"].append(y[:1]); outs["b"].append(y[1:])
    close(torch.cat(outs["a"]), want["a"], dtype, "token by token")
    close(torch.cat(outs["b"]), want["b"][:73], dtype, "two by two beside it")
    runner.cache.check()


# ------------------------------------------------------------------------------------------------ a toy architecture
@dataclass(frozen=True)
class ToyConfig:
    architecture: str
    hidden: int
    vocab: int
    inner: int
    heads: int
    head_dim: int
    eps: float
    order: tuple          # the schedule: (layer, cache, write) triples

    @classmethod
    def from_hf(cls, c):
        return cls(c["architectures"][0], c["hidden_size"], c["vocab_size"], c["inner"], c["heads"], c["head_dim"],
                   c["eps"], tuple(tuple(x) for x in c["order"]))

    def to_hf(self):
        return dict(architectures=[self.architecture], hidden_size=self.hidden, vocab_size=self.vocab, inner=self.inner,
                    heads=self.heads, head_dim=self.head_dim, eps=self.eps, order=[list(x) for x in self.order])


def toy_architecture():
    """Layer 0 and 2: attention (no position encoding in layer 2).  Layer 1: a running-mean mixer that keeps the sum of
    its inputs per request in a state slot.  The order layers run in comes from the configuration."""
    from mashbox_b200.cache.manager import StateNeed
    from mashbox_b200.config.registry import Architecture, register_architecture
    from mashbox_b200.parts import LayerRun, LayerSpec, ModelSpec, PartSpec, register
    from mashbox_b200.weights.loader import Want

    class RunningMean:
        """y_t = mean(h_0 .. h_t) W^T: state = the sum so far, one vector per request"""

        def __init__(self, hidden, prefix=""):
            self.D, self.name = hidden, prefix + "mean_proj.weight"

        def wants(self):
            return [Want(self.name, (self.D, self.D), "matrix")]

        def bind(self, tensors, env):
            self.w = tensors[self.name]

        def cache_need(self):
            return None

        def state_need(self):
            return StateNeed((self.D,), "float32")

        def prepare(self, ctx):
            pass

        def forward(self, ctx, h, run):
            state = ctx.cache.state[run.cache]
            out = torch.empty_like(h)
            for s in range(ctx.S):
                a, n, p0, slot = ctx.q_start[s], ctx.q_len[s], ctx.pos0[s], ctx.state_slots[s]
                sums = state[slot] + torch.cumsum(h[a:a + n].float(), 0)
                count = torch.arange(p0 + 1, p0 + n + 1, device=h.device, dtype=torch.float32)[:, None]
                out[a:a + n] = ctx.ops.linear((sums / count).to(h.dtype), self.w)
                state[slot] = sums[-1]
            return out, None

    register("mixer", "running_mean", RunningMean)

    def spec(c):
        norm = PartSpec("rms", width=c.hidden, eps=c.eps)
        ffn = PartSpec("swiglu", hidden=c.hidden, intermediate=c.inner)
        rope = PartSpec("rope", head_dim=c.head_dim, rotary_dim=c.head_dim, theta=10000.0)
        att = lambda pos: PartSpec("attention", hidden=c.hidden, heads=c.heads, kv_heads=c.heads, head_dim=c.head_dim,
                                   position=pos)
        mixers = [att(rope), PartSpec("running_mean", hidden=c.hidden), att(None)]
        return ModelSpec(hidden=c.hidden, vocab=c.vocab, embedding=PartSpec("table", vocab=c.vocab, hidden=c.hidden),
                         layers=[LayerSpec(prefix=f"blk.{i}.", block=PartSpec("prenorm", norm=norm, mixer=m, ffn=ffn))
                                 for i, m in enumerate(mixers)],
                         schedule=[LayerRun(layer=l, cache=ca, write=bool(w)) for l, ca, w in c.order],
                         final_norm=PartSpec("rms", width=c.hidden, eps=c.eps, name="output_norm.weight"),
                         head=PartSpec("linear", vocab=c.vocab, hidden=c.hidden, tied=True))

    def stored(c):
        D, A, F = c.hidden, c.heads * c.head_dim, c.inner
        out = {"token_embd.weight": ((c.vocab, D), "matrix"), "output_norm.weight": ((D,), "norm")}
        for i in range(3):
            p = f"blk.{i}."
            out[p + "attn_norm.weight"] = ((D,), "norm")
            out[p + "ffn_norm.weight"] = ((D,), "norm")
            for n, s in (("ffn_gate", (F, D)), ("ffn_up", (F, D)), ("ffn_down", (D, F))):
                out[p + n + ".weight"] = (s, "matrix")
            if i == 1:
                out[p + "mean_proj.weight"] = ((D, D), "matrix")
            else:
                for n, s in (("attn_q", (A, D)), ("attn_k", (A, D)), ("attn_v", (A, D)), ("attn_output", (D, A))):
                    out[p + n + ".weight"] = (s, "matrix")
        return out

    return register_architecture(Architecture("ToyMeanForCausalLM", ToyConfig, spec, lambda c: (lambda n: (n, None)),
                                              stored))


def toy_plain(cfg, W, tokens):
    """the toy model over one whole sequence with the plain functions, float64"""
    T = len(tokens)
    D, Hh, HD = cfg.hidden, cfg.heads, cfg.head_dim
    W = {k: v.double() for k, v in W.items()}
    pos = np.arange(T)
    fr = plain.rope_frequencies(10000.0, HD, None)
    x = W["token_embd.weight"][torch.tensor(tokens)]
    kept = {}
    for layer, cache, write in cfg.order:
        p = f"blk.{layer}."
        h = plain.rms_norm(x, W[p + "attn_norm.weight"], cfg.eps)
        if layer == 1:
            y = (torch.cumsum(h, 0) / torch.arange(1, T + 1)[:, None]) @ W[p + "mean_proj.weight"].T
        else:
            q = (h @ W[p + "attn_q.weight"].T).reshape(T, Hh, HD)
            k = (h @ W[p + "attn_k.weight"].T).reshape(T, Hh, HD)
            v = (h @ W[p + "attn_v.weight"].T).reshape(T, Hh, HD)
            if layer == 0:
                q, k = plain.rope_adjacent(q, pos, fr), plain.rope_adjacent(k, pos, fr)
            if write:
                kept[cache] = (k, v)
            k, v = kept[cache]
            y = plain.attention(q, k, v, HD ** -0.5) @ W[p + "attn_output.weight"].T
        x = x + y
        h = plain.rms_norm(x, W[p + "ffn_norm.weight"], cfg.eps)
        x = x + plain.swiglu(h, W[p + "ffn_gate.weight"], W[p + "ffn_up.weight"], W[p + "ffn_down.weight"])
    return (plain.rms_norm(x, W["output_norm.weight"], cfg.eps) @ W["token_embd.weight"].T).numpy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_with_state_a_layer_run_twice_and_a_shared_cache(tmp_path, dtype):
    from mashbox_b200.engine.replay import make_runner, run_step
    from mashbox_b200.weights.random_init import write_model_folder
    toy_architecture()
    # layer 0 (cache 0), the running mean (state under cache id 1), layer 0 AGAIN with a cache of its own (2), then
    # layer 2, which reads the keys layer 0 wrote on its first run and writes nothing
    cfg = ToyConfig("ToyMeanForCausalLM", hidden=48, vocab=131, inner=112, heads=3, head_dim=16, eps=1e-5,
                    order=((0, 0, 1), (1, 1, 1), (0, 2, 1), (2, 0, 0)))
    folder = write_model_folder(str(tmp_path / "toy"), cfg, 3, dtype=getattr(torch, dtype), std=0.12, norm_std=0.1,
                                std_by_name=(("token_embd", 1.0), ("attn_output", 0.03), ("ffn_down", 0.03),
                                             ("mean_proj", 0.03)))
    assert json.load(open(os.path.join(folder, "config.json")))["architectures"] == ["ToyMeanForCausalLM"]
    runner = make_runner(folder, dtype, 192, page_size=8)
    assert len(runner.cache.groups) == 1 and sorted(runner.cache.groups[0].cache_ids) == [0, 2]
    assert list(runner.cache.state) == [1] and tuple(runner.cache.state[1].shape[1:]) == (48,)
    W = plain.read_safetensors(os.path.join(folder, "model.safetensors"))
    rng = np.random.default_rng(0)
    a, b = rng.integers(0, 131, 90).tolist(), rng.integers(0, 131, 61).tolist()
    wa, wb = toy_plain(cfg, W, a), toy_plain(cfg, W, b)
    bar = lambda got, want, what: assert_logits(got, want, "float32", what) if dtype == "float32" else \
        close(torch.from_numpy(got), torch.from_numpy(want), "bfloat16", what)
    whole = run_step(runner, dict(step=0, entries=[dict(id="a", tokens=a, want=list(range(90)))], end=["a"])).numpy()
    bar(whole, wa, "toy, whole")
    # both requests in portions and single tokens, mixed; the state slot of "a" is used again by "b2" afterwards
    got = {"a": [], "b": []}
    cuts = {"a": [7, 2, 30, 1, 1, 19, 30], "b": [1, 1, 40, 2, 5, 12]}
    at = {"a": 0, "b": 0}
    toks = {"a": a, "b": b}
    for i in range(7):
        entries = []
        for r in ("a", "b"):
            if i < len(cuts[r]):
                n = cuts[r][i]
                entries.append(dict(id=r, tokens=toks[r][at[r]:at[r] + n], want=list(range(n))))
                at[r] += n
        out = run_step(runner, dict(step=i, entries=entries, end=[r for r in ("a", "b") if at[r] == len(toks[r]) and
                                                                 i == len(cuts[r]) - 1])).numpy()
        o = 0
        for e in entries:
            got[e["id"]].append(out[o:o + len(e["tokens"])])
            o += len(e["tokens"])
    bar(np.concatenate(got["a"]), wa, "toy, request a in portions")
    bar(np.concatenate(got["b"]), wb, "toy, request b in portions")
    again = run_step(runner, dict(step=0, entries=[dict(id="b2", tokens=b, want=[60])], end=["b2"])).numpy()
    bar(again, wb[60:], "toy, a state slot used again starts from zero")
    runner.cache.check()
