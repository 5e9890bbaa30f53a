"""-m gpu: two more kinds of part defined in this file and plugged in without a change to the framework's files: a
feed-forward that routes every token to one of several experts, and a position encoding with weights and arithmetic of
its own (a learned table added to queries and keys).  One layer uses them, the next one the framework's own rotary
encoding and dense feed-forward, so the choice is per layer.  They are toys that show the interfaces, no model of
anyone's; their arithmetic on the device is torch's, as a part under development would start out."""
import json
import os
from dataclasses import dataclass

import numpy as np
import pytest
import torch

from tests.plain import llama as plain
from tests.test_parts_gpu import close
from tests.tolerances import assert_logits

pytestmark = pytest.mark.gpu
PERIOD = 37          # the learned position table repeats after this many positions


@dataclass(frozen=True)
class RoutedConfig:
    architecture: str
    hidden: int
    vocab: int
    inner: int
    experts: int
    heads: int
    kv_heads: int
    head_dim: int
    eps: float

    @classmethod
    def from_hf(cls, c):
        return cls(c["architectures"][0], c["hidden_size"], c["vocab_size"], c["inner"], c["experts"], c["heads"],
                   c["kv_heads"], c["head_dim"], c["eps"])

    def to_hf(self):
        return dict(architectures=[self.architecture], hidden_size=self.hidden, vocab_size=self.vocab, inner=self.inner,
                    experts=self.experts, heads=self.heads, kv_heads=self.kv_heads, head_dim=self.head_dim, eps=self.eps)


def routed_architecture():
    from mashbox_b200.config.registry import Architecture, register_architecture
    from mashbox_b200.parts import LayerRun, LayerSpec, ModelSpec, PartSpec, register
    from mashbox_b200.weights.loader import Want

    class TopOneExperts:
        """y = p_e * expert_e(h) for e = argmax of the router's logits; p = softmax of the logits, in float32"""

        def __init__(self, hidden, intermediate, experts, prefix=""):
            self.D, self.F, self.E, self.p = hidden, intermediate, experts, prefix

        def wants(self):
            out = [Want(self.p + "router.weight", (self.E, self.D), "vector")]       # kept in float32
            for e in range(self.E):
                out += [Want(f"{self.p}expert.{e}.gate.weight", (self.F, self.D), "matrix"),
                        Want(f"{self.p}expert.{e}.up.weight", (self.F, self.D), "matrix"),
                        Want(f"{self.p}expert.{e}.down.weight", (self.D, self.F), "matrix")]
            return out

        def bind(self, tensors, env):
            self.router = tensors[self.p + "router.weight"]
            self.w = [tuple(tensors[f"{self.p}expert.{e}.{n}.weight"] for n in ("gate", "up", "down"))
                      for e in range(self.E)]

        def forward(self, ctx, h):
            ops = ctx.ops
            prob = torch.softmax(ops.linear(h.float().contiguous(), self.router), -1)
            top, choice = prob.max(-1)
            y = torch.zeros_like(h)
            for e, (wg, wu, wd) in enumerate(self.w):
                rows = (choice == e).nonzero()[:, 0]
                if rows.numel() == 0:
                    continue
                x = h[rows].contiguous()
                gu = torch.cat([ops.linear(x, wg), ops.linear(x, wu)], 1).contiguous()
                act = torch.empty((rows.numel(), self.F), dtype=h.dtype, device=h.device)
                ops.swiglu(gu, act)
                y[rows] = (ops.linear(act, wd).float() * top[rows, None]).to(h.dtype)
            return y, None

    class LearnedShift:
        """q and k of every head get table[position mod PERIOD] added: a position encoding that brings a tensor and
        does its own arithmetic on the fused q/k/v rows before they are stored"""

        def __init__(self, head_dim, prefix=""):
            self.HD, self.name = head_dim, prefix + "position_table.weight"

        def wants(self):
            return [Want(self.name, (PERIOD, self.HD), "vector")]

        def bind(self, tensors, env):
            self.table = tensors[self.name]

        def rotation(self):
            return None                     # no rotary table for the mixer's kernel: apply() does the work

        def apply(self, ctx, qkv, H, KV, HD):
            shift = self.table[(ctx.dev("positions") % PERIOD).long()]                  # (N, HD) float32
            qk = qkv[:, :(H + KV) * HD].view(qkv.shape[0], H + KV, HD)
            qk.copy_((qk.float() + shift[:, None, :]).to(qkv.dtype))

    register("feed_forward", "top_one_experts", TopOneExperts)
    register("position", "learned_shift", LearnedShift)

    def spec(c):
        norm = PartSpec("rms", width=c.hidden, eps=c.eps)
        att = lambda pos: PartSpec("attention", hidden=c.hidden, heads=c.heads, kv_heads=c.kv_heads,
                                   head_dim=c.head_dim, position=pos)
        layers = [LayerSpec(prefix="blk.0.", block=PartSpec(
                      "prenorm", norm=norm, mixer=att(PartSpec("learned_shift", head_dim=c.head_dim, prefix="blk.0.")),
                      ffn=PartSpec("top_one_experts", hidden=c.hidden, intermediate=c.inner, experts=c.experts))),
                  LayerSpec(prefix="blk.1.", block=PartSpec(
                      "prenorm", norm=norm,
                      mixer=att(PartSpec("rope", head_dim=c.head_dim, rotary_dim=c.head_dim // 2, theta=500.0,
                                         pairing="halves")),
                      ffn=PartSpec("swiglu", hidden=c.hidden, intermediate=c.inner)))]
        return ModelSpec(hidden=c.hidden, vocab=c.vocab, embedding=PartSpec("table", vocab=c.vocab, hidden=c.hidden),
                         layers=layers, schedule=[LayerRun(layer=i, cache=i, write=True) for i in range(2)],
                         final_norm=PartSpec("rms", width=c.hidden, eps=c.eps, name="output_norm.weight"),
                         head=PartSpec("linear", vocab=c.vocab, hidden=c.hidden, tied=False))

    def stored(c):
        D, F = c.hidden, c.inner
        A, B = c.heads * c.head_dim, c.kv_heads * c.head_dim
        out = {"token_embd.weight": ((c.vocab, D), "matrix"), "output.weight": ((c.vocab, D), "matrix"),
               "output_norm.weight": ((D,), "norm"), "blk.0.position_table.weight": ((PERIOD, c.head_dim), "vector"),
               "blk.0.router.weight": ((c.experts, D), "vector")}
        for i in range(2):
            p = f"blk.{i}."
            out[p + "attn_norm.weight"] = ((D,), "norm")
            out[p + "ffn_norm.weight"] = ((D,), "norm")
            for n, s in (("attn_q", (A, D)), ("attn_k", (B, D)), ("attn_v", (B, D)), ("attn_output", (D, A))):
                out[p + n + ".weight"] = (s, "matrix")
        for e in range(c.experts):
            for n, s in (("gate", (F, D)), ("up", (F, D)), ("down", (D, F))):
                out[f"blk.0.expert.{e}.{n}.weight"] = (s, "matrix")
        for n, s in (("ffn_gate", (F, D)), ("ffn_up", (F, D)), ("ffn_down", (D, F))):
            out["blk.1." + n + ".weight"] = (s, "matrix")
        return out

    return register_architecture(Architecture("ToyRoutedForCausalLM", RoutedConfig, spec,
                                              lambda c: (lambda n: (n, None)), stored))


def routed_plain(cfg, W, tokens):
    """the toy model over one whole sequence with the plain functions, float64 -> (logits, smallest router margin)"""
    T = len(tokens)
    D, Hh, KV, HD = cfg.hidden, cfg.heads, cfg.kv_heads, cfg.head_dim
    W = {k: v.double() for k, v in W.items()}
    pos = np.arange(T)
    x = W["token_embd.weight"][torch.tensor(tokens)]
    margin = float("inf")
    for layer in range(2):
        p = f"blk.{layer}."
        h = plain.rms_norm(x, W[p + "attn_norm.weight"], cfg.eps)
        q = (h @ W[p + "attn_q.weight"].T).reshape(T, Hh, HD)
        k = (h @ W[p + "attn_k.weight"].T).reshape(T, KV, HD)
        v = (h @ W[p + "attn_v.weight"].T).reshape(T, KV, HD)
        if layer == 0:
            shift = W[p + "position_table.weight"][torch.tensor(pos % PERIOD)][:, None, :]
            q, k = q + shift, k + shift
        else:
            fr = plain.rope_frequencies(500.0, HD // 2, None)
            q, k = plain.rope_halves(q, pos, fr), plain.rope_halves(k, pos, fr)
        x = x + plain.attention(q, k, v, HD ** -0.5).reshape(T, Hh * HD) @ W[p + "attn_output.weight"].T
        h = plain.rms_norm(x, W[p + "ffn_norm.weight"], cfg.eps)
        if layer == 0:
            logits = h @ W[p + "router.weight"].T
            prob = torch.softmax(logits, -1)
            best = torch.sort(logits, -1, descending=True).values
            margin = min(margin, float((best[:, 0] - best[:, 1]).min()))
            top, choice = prob.max(-1)
            y = torch.zeros_like(x)
            for e in range(cfg.experts):
                rows = choice == e
                y[rows] = plain.swiglu(h[rows], W[f"{p}expert.{e}.gate.weight"], W[f"{p}expert.{e}.up.weight"],
                                       W[f"{p}expert.{e}.down.weight"]) * top[rows, None]
            x = x + y
        else:
            x = x + plain.swiglu(h, W[p + "ffn_gate.weight"], W[p + "ffn_up.weight"], W[p + "ffn_down.weight"])
    return (plain.rms_norm(x, W["output_norm.weight"], cfg.eps) @ W["output.weight"].T).numpy(), margin


ROUTED = RoutedConfig("ToyRoutedForCausalLM", hidden=80, vocab=211, inner=96, experts=3, heads=4, kv_heads=2, head_dim=32,
                      eps=1e-6)
SEED = 11
SCALES = (("token_embd", 1.0), ("attn_output", 0.03), ("down", 0.03), ("router", 1.0), ("position_table", 0.5))


def routed_folder(path, dtype):
    from mashbox_b200.weights.random_init import write_model_folder
    routed_architecture()
    return write_model_folder(str(path), ROUTED, SEED, dtype=getattr(torch, dtype), std=0.11, norm_std=0.1,
                              std_by_name=SCALES)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_routed_feed_forward_and_learned_position_encoding_per_layer(tmp_path, dtype):
    from mashbox_b200.engine.replay import make_runner, run_step
    folder = routed_folder(tmp_path / "routed", dtype)
    assert json.load(open(os.path.join(folder, "config.json")))["experts"] == 3
    runner = make_runner(folder, dtype, 256, page_size=8, options={"no_graphs": True})     # the toy reads its routing on the host
    W = plain.read_safetensors(os.path.join(folder, "model.safetensors"))
    rng = np.random.default_rng(1)
    a, b = rng.integers(0, 211, 100).tolist(), rng.integers(0, 211, 45).tolist()
    (wa, ma), (wb, mb) = routed_plain(ROUTED, W, a), routed_plain(ROUTED, W, b)
    # a router decision within rounding of a tie would make this a test of luck: the seed is chosen so that none is
    assert min(ma, mb) > 0.15, (ma, mb)
    bar = lambda got, want, what: assert_logits(got, want, "float32", what) if dtype == "float32" else \
        close(torch.from_numpy(got), torch.from_numpy(want), "bfloat16", what)
    whole = run_step(runner, dict(step=0, entries=[dict(id="a", tokens=a, want=list(range(100)))], end=["a"])).numpy()
    bar(whole, wa, "routed toy, whole")
    got = {"a": [], "b": []}
    cuts = {"a": [50, 2, 1, 1, 30, 16], "b": [3, 1, 1, 38, 2]}
    at, toks = {"a": 0, "b": 0}, {"a": a, "b": b}
    for i in range(6):
        entries = []
        for r in ("a", "b"):
            if i < len(cuts[r]):
                n = cuts[r][i]
                entries.append(dict(id=r, tokens=toks[r][at[r]:at[r] + n], want=list(range(n))))
                at[r] += n
        out = run_step(runner, dict(step=i, entries=entries, end=[])).numpy()
        o = 0
        for e in entries:
            got[e["id"]].append(out[o:o + len(e["tokens"])])
            o += len(e["tokens"])
    bar(np.concatenate(got["a"]), wa, "routed toy, request a in portions beside b")
    bar(np.concatenate(got["b"]), wb, "routed toy, request b in portions beside a")
    runner.cache.check()


# ---------------------------------------------------------------------------------------- two head sizes in one model
@dataclass(frozen=True)
class TwoSizesConfig:
    architecture: str
    hidden: int
    vocab: int
    inner: int
    kv_heads: int
    groups: int
    head_dims: tuple
    eps: float

    @classmethod
    def from_hf(cls, c):
        return cls(c["architectures"][0], c["hidden_size"], c["vocab_size"], c["inner"], c["kv_heads"], c["groups"],
                   tuple(c["head_dims"]), c["eps"])

    def to_hf(self):
        return dict(architectures=[self.architecture], hidden_size=self.hidden, vocab_size=self.vocab, inner=self.inner,
                    kv_heads=self.kv_heads, groups=self.groups, head_dims=list(self.head_dims), eps=self.eps)


def two_sizes_architecture():
    from mashbox_b200.config.registry import Architecture, register_architecture
    from mashbox_b200.parts import LayerRun, LayerSpec, ModelSpec, PartSpec

    def spec(c):
        norm = PartSpec("rms", width=c.hidden, eps=c.eps)
        ffn = PartSpec("swiglu", hidden=c.hidden, intermediate=c.inner)
        layers = []
        for i, hd in enumerate(c.head_dims):
            rope = PartSpec("rope", head_dim=hd, rotary_dim=hd, theta=10000.0)
            att = PartSpec("attention", hidden=c.hidden, heads=c.kv_heads * c.groups, kv_heads=c.kv_heads, head_dim=hd,
                           position=rope)
            layers.append(LayerSpec(f"blk.{i}.", PartSpec("prenorm", norm=norm, mixer=att, ffn=ffn)))
        return ModelSpec(hidden=c.hidden, vocab=c.vocab, embedding=PartSpec("table", vocab=c.vocab, hidden=c.hidden),
                         layers=layers, schedule=[LayerRun(layer=i, cache=i, write=True) for i in range(len(layers))],
                         final_norm=PartSpec("rms", width=c.hidden, eps=c.eps, name="output_norm.weight"),
                         head=PartSpec("linear", vocab=c.vocab, hidden=c.hidden, tied=True))

    def stored(c):
        D, F = c.hidden, c.inner
        out = {"token_embd.weight": ((c.vocab, D), "matrix"), "output_norm.weight": ((D,), "norm")}
        for i, hd in enumerate(c.head_dims):
            p, A, B = f"blk.{i}.", c.kv_heads * c.groups * hd, c.kv_heads * hd
            out[p + "attn_norm.weight"] = ((D,), "norm")
            out[p + "ffn_norm.weight"] = ((D,), "norm")
            for n, s in (("attn_q", (A, D)), ("attn_k", (B, D)), ("attn_v", (B, D)), ("attn_output", (D, A)),
                         ("ffn_gate", (F, D)), ("ffn_up", (F, D)), ("ffn_down", (D, F))):
                out[p + n + ".weight"] = (s, "matrix")
        return out

    return register_architecture(Architecture("ToyTwoSizesForCausalLM", TwoSizesConfig, spec,
                                              lambda c: (lambda n: (n, None)), stored))


def two_sizes_plain(cfg, W, tokens):
    T = len(tokens)
    W = {k: v.double() for k, v in W.items()}
    pos = np.arange(T)
    x = W["token_embd.weight"][torch.tensor(tokens)]
    for i, hd in enumerate(cfg.head_dims):
        p, Hh = f"blk.{i}.", cfg.kv_heads * cfg.groups
        fr = plain.rope_frequencies(10000.0, hd, None)
        h = plain.rms_norm(x, W[p + "attn_norm.weight"], cfg.eps)
        q = plain.rope_adjacent((h @ W[p + "attn_q.weight"].T).reshape(T, Hh, hd), pos, fr)
        k = plain.rope_adjacent((h @ W[p + "attn_k.weight"].T).reshape(T, cfg.kv_heads, hd), pos, fr)
        v = (h @ W[p + "attn_v.weight"].T).reshape(T, cfg.kv_heads, hd)
        x = x + plain.attention(q, k, v, hd ** -0.5) @ W[p + "attn_output.weight"].T
        h = plain.rms_norm(x, W[p + "ffn_norm.weight"], cfg.eps)
        x = x + plain.swiglu(h, W[p + "ffn_gate.weight"], W[p + "ffn_up.weight"], W[p + "ffn_down.weight"])
    return (plain.rms_norm(x, W["output_norm.weight"], cfg.eps) @ W["token_embd.weight"].T).numpy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_layers_of_two_head_sizes_in_one_model(tmp_path, dtype):
    """layers with the same groups, kv heads and window but heads of 128, 32 and 64: each head size has its own plan of
    attention work in a step (tiles of 256 packed rows on the tcgen05 kernel at 128 and 64, of 64 rows on the mma.sync
    kernel at 32; a plan made for one and used for the other would leave rows out) and its own cache group"""
    from mashbox_b200.engine.replay import make_runner, run_step
    from mashbox_b200.weights.random_init import write_model_folder
    two_sizes_architecture()
    cfg = TwoSizesConfig("ToyTwoSizesForCausalLM", hidden=128, vocab=157, inner=160, kv_heads=2, groups=2,
                         head_dims=(128, 32, 64), eps=1e-5)
    folder = write_model_folder(str(tmp_path / "two"), cfg, 9, dtype=getattr(torch, dtype), std=0.08, norm_std=0.1,
                                std_by_name=(("token_embd", 1.0), ("attn_output", 0.03), ("ffn_down", 0.03)))
    runner = make_runner(folder, dtype, 1024, page_size=16)
    assert sorted(g.need.tensors[0] for g in runner.cache.groups) == [(2, 32), (2, 64), (2, 128)]
    W = plain.read_safetensors(os.path.join(folder, "model.safetensors"))
    rng = np.random.default_rng(4)
    a, b = rng.integers(0, 157, 300).tolist(), rng.integers(0, 157, 41).tolist()
    wa, wb = two_sizes_plain(cfg, W, a), two_sizes_plain(cfg, W, b)
    bar = lambda got, want, what: assert_logits(got, want, "float32", what) if dtype == "float32" else \
        close(torch.from_numpy(got), torch.from_numpy(want), "bfloat16", what)
    # a long portion (prompt-form tiles of 256 packed rows on tcgen05 at both head sizes) beside single tokens and a
    # short portion of another request
    out = run_step(runner, dict(step=0, entries=[dict(id="a", tokens=a[:280], want=[0, 100, 279]),
                                                 dict(id="b", tokens=b[:30], want=[29])], end=[])).numpy()
    bar(out[:3], wa[[0, 100, 279]], "two head sizes, portion of a")
    bar(out[3:], wb[29:30], "two head sizes, portion of b")
    got_a, got_b = [], []
    for i in range(11):
        entries = [dict(id="a", tokens=[a[280 + i]], want=[0]), dict(id="b", tokens=[b[30 + i]], want=[0])]
        o = run_step(runner, dict(step=1 + i, entries=entries, end=[])).numpy()
        got_a.append(o[0])
        got_b.append(o[1])
    bar(np.stack(got_a), wa[280:291], "two head sizes, a decoded")
    bar(np.stack(got_b), wb[30:41], "two head sizes, b decoded")
    runner.cache.check()
