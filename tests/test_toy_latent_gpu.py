"""-m gpu: a third toy, defined here and plugged in without a change to the framework's files, that leans on three
seams of the framework at once:

  * a mixer that keeps ONE latent vector per position (no keys and values) in pages of its own layout, beside an
    attention layer whose pages hold keys and values: two cache groups with different per-position tensors;
  * the same mixer works on blocks of GRID positions, so the scheduler must end every portion of a prompt on a
    multiple of GRID unless it reaches the prompt's end (the mixer checks where its portions start);
  * a pre-norm block whose two norms differ (their eps), given as norm1 / norm2 of the block's own spec.

It runs through Engine.generate (scheduler, step function, cache manager, sampler) against a plain float64 loop.  A toy
that shows the interfaces, no model of anyone's; its arithmetic on the device is torch's.
"""
from dataclasses import dataclass

import numpy as np
import pytest
import torch

from tests.plain import llama as plain

pytestmark = pytest.mark.gpu
GRID = 4
RANK = 24


@dataclass(frozen=True)
class LatentConfig:
    architecture: str
    hidden: int
    vocab: int
    inner: int
    heads: int
    head_dim: int
    eps1: float
    eps2: float

    @classmethod
    def from_hf(cls, c):
        return cls(c["architectures"][0], c["hidden_size"], c["vocab_size"], c["inner"], c["heads"], c["head_dim"],
                   c["eps1"], c["eps2"])

    def to_hf(self):
        return dict(architectures=[self.architecture], hidden_size=self.hidden, vocab_size=self.vocab, inner=self.inner,
                    heads=self.heads, head_dim=self.head_dim, eps1=self.eps1, eps2=self.eps2)


STARTS = []         # (first position, tokens) of every portion the latent mixer saw


def latent_architecture():
    from mashbox_b200.cache.manager import CacheNeed
    from mashbox_b200.config.registry import Architecture, register_architecture
    from mashbox_b200.parts import LayerRun, LayerSpec, ModelSpec, PartSpec, register
    from mashbox_b200.weights.loader import Want

    class LatentMean:
        """c_t = h_t Wc^T (RANK wide) is kept per position; y_t = (mean of c_s over the positions s <= t of t's block
        and of every block before it) Wu^T.  It reads the older latents back from its pages through the block table."""
        portion_alignment = GRID

        def __init__(self, hidden, rank, prefix=""):
            self.D, self.R, self.p = hidden, rank, prefix

        def wants(self):
            return [Want(self.p + "latent_down.weight", (self.R, self.D), "matrix"),
                    Want(self.p + "latent_up.weight", (self.D, self.R), "matrix")]

        def bind(self, tensors, env):
            self.wc, self.wu = tensors[self.p + "latent_down.weight"], tensors[self.p + "latent_up.weight"]

        def cache_need(self):
            return CacheNeed("full", ((1, self.R),))

        def state_need(self):
            return None

        def prepare(self, ctx):
            pass

        def forward(self, ctx, h, run):
            group, pool = ctx.cache.layer_cache(run.cache)              # (pages, 1, page, RANK)
            page = ctx.cache.page_size
            table = torch.from_numpy(group.table).to(h.device).long()
            c = ctx.ops.linear(h, self.wc)
            out = torch.empty((h.shape[0], self.R), dtype=torch.float32, device=h.device)
            for s in range(ctx.S):
                a, n, p0, row = ctx.q_start[s], ctx.q_len[s], ctx.pos0[s], ctx.rows[s]
                STARTS.append((p0, n))
                pos = torch.arange(p0, p0 + n, device=h.device)
                if run.write:
                    pool[table[row, pos // page], 0, pos % page] = c[a:a + n]
                old = torch.arange(0, p0 + n, device=h.device)
                kept = pool[table[row, old // page], 0, old % page].float()          # this portion's own included
                out[a:a + n] = torch.cumsum(kept, 0)[p0:] / (pos + 1).float()[:, None]
            return ctx.ops.linear(out.to(h.dtype), self.wu), None

    register("mixer", "latent_mean", LatentMean)

    def spec(c):
        n1, n2 = PartSpec("rms", width=c.hidden, eps=c.eps1), PartSpec("rms", width=c.hidden, eps=c.eps2)
        ffn = PartSpec("swiglu", hidden=c.hidden, intermediate=c.inner)
        rope = PartSpec("rope", head_dim=c.head_dim, rotary_dim=c.head_dim, theta=10000.0)
        att = PartSpec("attention", hidden=c.hidden, heads=c.heads, kv_heads=1, head_dim=c.head_dim, position=rope)
        lat = PartSpec("latent_mean", hidden=c.hidden, rank=RANK)
        layers = [LayerSpec("blk.0.", PartSpec("prenorm", norm1=n1, norm2=n2, mixer=lat, ffn=ffn)),
                  LayerSpec("blk.1.", PartSpec("prenorm", norm1=n2, norm2=n1, mixer=att, ffn=ffn))]
        return ModelSpec(hidden=c.hidden, vocab=c.vocab, embedding=PartSpec("table", vocab=c.vocab, hidden=c.hidden),
                         layers=layers, schedule=[LayerRun(layer=i, cache=i, write=True) for i in range(2)],
                         final_norm=PartSpec("rms", width=c.hidden, eps=c.eps1, name="output_norm.weight"),
                         head=PartSpec("linear", vocab=c.vocab, hidden=c.hidden, tied=True))

    def stored(c):
        D, F, A = c.hidden, c.inner, c.heads * c.head_dim
        out = {"token_embd.weight": ((c.vocab, D), "matrix"), "output_norm.weight": ((D,), "norm"),
               "blk.0.latent_down.weight": ((RANK, D), "matrix"), "blk.0.latent_up.weight": ((D, RANK), "matrix")}
        for i in range(2):
            p = f"blk.{i}."
            out[p + "attn_norm.weight"] = ((D,), "norm")
            out[p + "ffn_norm.weight"] = ((D,), "norm")
            for n, s in (("ffn_gate", (F, D)), ("ffn_up", (F, D)), ("ffn_down", (D, F))):
                out[p + n + ".weight"] = (s, "matrix")
        for n, s in (("attn_q", (A, D)), ("attn_k", (c.head_dim, D)), ("attn_v", (c.head_dim, D)), ("attn_output", (D, A))):
            out["blk.1." + n + ".weight"] = (s, "matrix")
        return out

    return register_architecture(Architecture("ToyLatentForCausalLM", LatentConfig, spec,
                                              lambda c: (lambda n: (n, None)), stored))


def latent_plain(cfg, W, tokens):
    """the toy over one whole sequence, float64 -> logits (T, V)"""
    T, D, Hh, HD = len(tokens), cfg.hidden, cfg.heads, cfg.head_dim
    W = {k: v.double() for k, v in W.items()}
    x = W["token_embd.weight"][torch.tensor(tokens)]
    h = plain.rms_norm(x, W["blk.0.attn_norm.weight"], cfg.eps1)
    c = h @ W["blk.0.latent_down.weight"].T
    x = x + (torch.cumsum(c, 0) / torch.arange(1, T + 1)[:, None]) @ W["blk.0.latent_up.weight"].T
    h = plain.rms_norm(x, W["blk.0.ffn_norm.weight"], cfg.eps2)
    x = x + plain.swiglu(h, W["blk.0.ffn_gate.weight"], W["blk.0.ffn_up.weight"], W["blk.0.ffn_down.weight"])
    h = plain.rms_norm(x, W["blk.1.attn_norm.weight"], cfg.eps2)
    fr = plain.rope_frequencies(10000.0, HD, None)
    q = plain.rope_adjacent((h @ W["blk.1.attn_q.weight"].T).reshape(T, Hh, HD), np.arange(T), fr)
    k = plain.rope_adjacent((h @ W["blk.1.attn_k.weight"].T).reshape(T, 1, HD), np.arange(T), fr)
    v = (h @ W["blk.1.attn_v.weight"].T).reshape(T, 1, HD)
    x = x + plain.attention(q, k, v, HD ** -0.5) @ W["blk.1.attn_output.weight"].T
    h = plain.rms_norm(x, W["blk.1.ffn_norm.weight"], cfg.eps1)
    x = x + plain.swiglu(h, W["blk.1.ffn_gate.weight"], W["blk.1.ffn_up.weight"], W["blk.1.ffn_down.weight"])
    return (plain.rms_norm(x, W["output_norm.weight"], cfg.eps1) @ W["token_embd.weight"].T).numpy()


def test_latent_cache_portion_grid_and_two_norms_through_generate(tmp_path):
    import os

    from mashbox_b200.engine.engine import Engine
    from mashbox_b200.weights.random_init import write_model_folder
    latent_architecture()
    cfg = LatentConfig("ToyLatentForCausalLM", hidden=40, vocab=97, inner=72, heads=3, head_dim=16, eps1=1e-6, eps2=0.3)
    folder = write_model_folder(str(tmp_path / "latent"), cfg, 5, dtype=torch.float32, std=0.15, norm_std=0.1,
                                std_by_name=(("token_embd", 1.0), ("attn_output", 0.05), ("ffn_down", 0.05),
                                             ("latent_up", 0.05)))
    eng = Engine.from_folder(folder, dtype="float32", page_size=8, max_tokens=512, max_requests=4,
                             max_tokens_per_step=22, chunk=14)
    cache = eng.cache
    assert eng.scheduler.align == GRID and not eng.runner.use_graphs        # the toy reads the batch on the host
    assert sorted(tuple(g.need.tensors) for g in cache.groups) == [((1, 16), (1, 16)), ((1, RANK),)]
    assert sorted(len(g.pools) for g in cache.groups) == [1, 2]
    W = plain.read_safetensors(os.path.join(folder, "model.safetensors"))
    rng = np.random.default_rng(2)
    prompts = [rng.integers(0, 97, n).tolist() for n in (37, 9, 50, 3)]
    STARTS.clear()
    out = eng.generate(prompts, max_new=6)
    # every portion the mixer saw began on the grid, or was a decoded token / the rest of a prompt after such a portion
    cuts = [(p0, n) for p0, n in STARTS if n > 1]
    assert len(cuts) >= 8 and all(p0 % GRID == 0 for p0, n in cuts)
    assert any((p0 + n) % GRID for p0, n in cuts)                            # ends of prompts are off the grid
    for p, ids in zip(prompts, out["ids"]):
        seq = list(p)
        for t in ids:                                                        # greedy, one token at a time, whole sequences
            lg = latent_plain(cfg, W, seq)[-1]
            best = np.sort(lg)[-2:]
            assert int(np.argmax(lg)) == t or best[1] - best[0] < 1e-4, (len(seq), t, int(np.argmax(lg)))
            seq.append(t)
    # eps2 = 0.3 is large enough that a block that used one norm spec for both norms would show
    swapped = LatentConfig(cfg.architecture, cfg.hidden, cfg.vocab, cfg.inner, cfg.heads, cfg.head_dim, cfg.eps2, cfg.eps1)
    a, b = latent_plain(cfg, W, prompts[0]), latent_plain(swapped, W, prompts[0])
    assert np.abs(a - b).max() > 0.05 * np.abs(a).max()
    cache.check()
    assert all(f == cache.num_pages for f in cache.free_pages())
