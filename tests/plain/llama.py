"""Plain, slow implementation of the Llama-3 dense decoder: whole sequences, no cache, one function per part.

It is the oracle the engine is compared with.  It shares no code with ``mashbox_b200``: it has its own
safetensors reader, reads config.json keys itself and works on CPU tensors in float64 (inputs that the
reference computes in float32 -- rotation angles -- are first formed in float32, then widened, so that the
oracle answers the same question as a float32 engine and not a slightly different one).

Every function is written from the formulas of mashbox-labs/mashbox and cites the file and lines (paths within
that project).  The reference's model module needs JAX and cannot be imported here, so this file rests on the
formulas; it is anchored on the reference's committed Hugging Face fixtures (transformers' own logits), see
tests/golden/make_golden.py and tests/test_plain.py.
"""
import json
import math
import os
import struct

import numpy as np
import torch

F64 = torch.float64


# ------------------------------------------------------------------------------------------------ files
def read_safetensors(path):
    """-> {name: float64 tensor}.  Format as src/mashbox/hf/source.py:58-69, 88-99: 8-byte little-endian header
    length, a JSON header {name: {dtype, shape, data_offsets}}, then the data; BF16, F16 and F32 only."""
    with open(path, "rb") as fh:
        (n,) = struct.unpack("<Q", fh.read(8))
        header = json.loads(fh.read(n))
        base = 8 + n
        blob = np.fromfile(fh, dtype=np.uint8)
    header.pop("__metadata__", None)
    out = {}
    for name, t in header.items():
        b, e = t["data_offsets"]
        raw = blob[b:e]
        shape = tuple(t["shape"])
        if t["dtype"] == "F32":
            a = raw.view(np.float32).astype(np.float64)
        elif t["dtype"] == "F16":
            a = raw.view(np.float16).astype(np.float64)
        elif t["dtype"] == "BF16":      # src/mashbox/hf/adapter.py:238-239: bf16 bits << 16 are the float32 value
            a = (raw.view(np.uint16).astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        else:
            raise ValueError(f"{name}: dtype {t['dtype']}")
        out[name] = torch.from_numpy(a.reshape(shape).copy())
    assert base > 8
    return out


def read_model(folder):
    """-> (config dict, {HF tensor name: float64 tensor})"""
    cfg = json.load(open(os.path.join(folder, "config.json")))
    return cfg, read_safetensors(os.path.join(folder, "model.safetensors"))


# ------------------------------------------------------------------------------------------------ config
def sizes(cfg):
    """The sizes and constants of config.json with the reference's defaults (src/mashbox/hf/adapter.py:97-131):
    KV defaults to H, head_dim to hidden/H, rms_norm_eps to 1e-6; theta and scaling from rope_parameters
    (transformers 5) or rope_theta + rope_scaling (adapter.py:83-90)."""
    H = int(cfg["num_attention_heads"])
    D = int(cfg["hidden_size"])
    rp = cfg.get("rope_parameters") or {}
    theta = float(rp.get("rope_theta", cfg.get("rope_theta", 10000.0)))
    sc = cfg.get("rope_scaling") or None
    if rp.get("rope_type") not in (None, "default"):
        sc = rp
    return dict(L=int(cfg["num_hidden_layers"]), D=D, H=H, KV=int(cfg.get("num_key_value_heads") or H),
                HD=int(cfg.get("head_dim") or D // H), F=int(cfg["intermediate_size"]),
                eps=float(cfg.get("rms_norm_eps", 1e-6)), theta=theta, scaling=sc,
                tie=bool(cfg.get("tie_word_embeddings", False)))


# ------------------------------------------------------------------------------------------------ parts
def permute_rows(w, n_head):
    """The q/k row permutation applied to Hugging Face weights so that the rotation acts on adjacent pairs:
    rows (n_head, 2, HD/2) -> (n_head, HD/2, 2).  src/mashbox/hf/adapter.py:223-225."""
    shape = w.shape
    return w.reshape((n_head, 2, shape[0] // n_head // 2) + tuple(shape[1:])).transpose(1, 2).reshape(shape)


def llama3_factors(theta, dim, sc):
    """One divisor per rotated pair for rope_type llama3.  src/mashbox/hf/adapter.py:162-179."""
    freqs = 1.0 / (np.float32(theta) ** (np.arange(0, dim, 2, dtype=np.float32) / np.float32(dim)))
    factor = float(sc.get("factor", 8.0))
    lo, hi = float(sc.get("low_freq_factor", 1.0)), float(sc.get("high_freq_factor", 4.0))
    old = float(sc.get("original_max_position_embeddings", 8192))
    out = []
    for f in freqs:
        w = 2 * math.pi / float(f)
        if w < old / hi:
            out.append(1.0)
        elif w > old / lo:
            out.append(factor)
        else:
            s = (old / w - lo) / (hi - lo)
            out.append(1.0 / ((1 - s) / factor + s))
    return np.asarray(out, np.float32)


def rope_frequencies(theta, rd, scaling):
    """float32 angle per position step for each rotated pair: inv_i = theta^(-2i/RD) (src/mashbox/gguf/archs/
    dense.py:302), divided by the llama3 factors when there are any (dense.py:316), times 1/factor for linear
    scaling (dense.py:93-94, 317)."""
    inv = (1.0 / (np.float32(theta) ** (np.arange(0, rd, 2, dtype=np.int64).astype(np.float32) / np.float32(rd)))
           ).astype(np.float32)
    kind = (scaling or {}).get("rope_type", (scaling or {}).get("type"))
    if kind in (None, "default"):
        return inv
    if kind == "linear":
        return (inv * np.float32(1.0 / float(scaling["factor"]))).astype(np.float32)
    if kind == "llama3":
        return (inv / llama3_factors(theta, rd, scaling)).astype(np.float32)
    raise ValueError(kind)


def rope_adjacent(x, positions, freqs):
    """Rotate adjacent pairs (x[2i], x[2i+1]) by angle pos * freq_i; dims past 2*len(freqs) pass through.
    src/mashbox/gguf/archs/dense.py:280-290 (NORM form), angles dense.py:317-318 (float32 product).
    x (T, heads, HD), positions (T,) ints."""
    rd = 2 * len(freqs)
    ang = (np.asarray(positions, np.float32)[:, None] * np.asarray(freqs, np.float32)[None, :]).astype(np.float32)
    ang = torch.from_numpy(ang.astype(np.float64))
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., 0:rd:2], x[..., 1:rd:2]
    rot = torch.stack([a * cos - b * sin, a * sin + b * cos], -1).reshape(x.shape[:-1] + (rd,))
    return torch.cat([rot, x[..., rd:]], -1)


def rope_halves(x, positions, freqs):
    """Rotate (x[i], x[i + RD/2]) -- the NEOX form of src/mashbox/gguf/archs/dense.py:284-286; equal to the
    adjacent form on permuted rows (that equality is what the permutation is for)."""
    rd = 2 * len(freqs)
    ang = (np.asarray(positions, np.float32)[:, None] * np.asarray(freqs, np.float32)[None, :]).astype(np.float32)
    ang = torch.from_numpy(ang.astype(np.float64))
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :rd // 2], x[..., rd // 2:rd]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., rd:]], -1)


def rms_norm(x, w, eps):
    """x * rsqrt(mean(x^2) + eps) * w, weight as stored.  src/mashbox/gguf/archs/qwen35.py:343-346."""
    return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w


def attention(q, k, v, scale, window=None, positions=None):
    """Causal grouped-query attention over one whole sequence.  q (T, H, HD), k, v (T, KV, HD); query head h reads
    kv head h // G (src/mashbox/gguf/archs/dense.py:347); scores * scale, masked to -1e30, softmax, weighted sum
    (src/mashbox/runtime/attention.py:58-62); mask key <= query (dense.py:321).  window w (other layer kinds keep
    the last w positions, src/mashbox/runtime/kvcache.py:21-23): key > query - w as well."""
    T, H, HD = q.shape
    KV = k.shape[1]
    G = H // KV
    pos = torch.arange(T) if positions is None else torch.as_tensor(positions)
    s = torch.einsum("tkgd,skd->kgts", q.reshape(T, KV, G, HD), k) * scale
    mask = pos[:, None] >= pos[None, :]
    if window is not None:
        mask = mask & (pos[None, :] > pos[:, None] - window)
    s = torch.where(mask[None, None], s, torch.full_like(s, -1e30))
    p = torch.softmax(s, -1)
    return torch.einsum("kgts,skd->tkgd", p, v).reshape(T, H * HD)


def swiglu(h, wg, wu, wd):
    """(silu(h Wg^T) * (h Wu^T)) Wd^T, silu(z) = z * sigmoid(z).  src/mashbox/gguf/archs/dense.py:356-357."""
    g = h @ wg.T
    return ((g * torch.sigmoid(g)) * (h @ wu.T)) @ wd.T


def linear(x, w, b=None):
    """x W^T (+ b).  src/mashbox/ops/__init__.py:594-595; bias src/mashbox/gguf/archs/dense.py:335-337."""
    y = x @ w.T
    return y if b is None else y + b


def _same(t):
    return t


def round_bf16(t):
    """round to bfloat16 and widen again: what holding a tensor in bfloat16 does to its values"""
    return t.to(torch.float32).to(torch.bfloat16).to(F64)


def block(x, W, l, c, freqs, positions, held=_same):
    """One pre-norm residual block: x += attn(ln1(x)); x += ffn(ln2(x)).  src/mashbox/gguf/archs/dense.py:339-357.
    W holds Hugging Face names; q/k rows are permuted here as the loader of the reference does.  `held` is applied to
    every tensor the reference holds in its activation dtype (dense.py:335-357: the results of rms, of every matmul,
    of the rotation and of silu*up are cast to `act`; biases are added in float32 before the cast of q, k, v and
    after it for the output); the identity gives the exact model, round_bf16 a model of bfloat16 storage."""
    p = f"model.layers.{l}."
    T = x.shape[0]
    H, KV, HD = c["H"], c["KV"], c["HD"]
    bias = lambda n: W.get(p + n)
    plus = lambda y, b: y if b is None else y + b
    h = held(rms_norm(x, W[p + "input_layernorm.weight"], c["eps"]))
    wq, wk = permute_rows(W[p + "self_attn.q_proj.weight"], H), permute_rows(W[p + "self_attn.k_proj.weight"], KV)
    bq, bk = bias("self_attn.q_proj.bias"), bias("self_attn.k_proj.bias")
    bq = None if bq is None else permute_rows(bq, H)
    bk = None if bk is None else permute_rows(bk, KV)
    q = plus(held(linear(h, wq)), bq).reshape(T, H, HD)
    k = plus(held(linear(h, wk)), bk).reshape(T, KV, HD)
    v = held(plus(held(linear(h, W[p + "self_attn.v_proj.weight"])), bias("self_attn.v_proj.bias"))).reshape(T, KV, HD)
    q, k = held(rope_adjacent(q, positions, freqs)), held(rope_adjacent(k, positions, freqs))
    o = held(attention(q, k, v, HD ** -0.5, window=c.get("window"), positions=positions))
    x = x + plus(held(linear(o, W[p + "self_attn.o_proj.weight"])), bias("self_attn.o_proj.bias"))
    h = held(rms_norm(x, W[p + "post_attention_layernorm.weight"], c["eps"]))
    g = held(linear(h, W[p + "mlp.gate_proj.weight"]))
    u = held(linear(h, W[p + "mlp.up_proj.weight"]))
    a = held(g * torch.sigmoid(g) * u)                                  # dense.py:356
    return x + held(linear(a, W[p + "mlp.down_proj.weight"]))


def head(x, W, c, held=_same):
    """logits = rms(x, norm) W_head^T; the head is the embedding when tied.  src/mashbox/gguf/archs/dense.py:386-390,
    tie dense.py:129.  The logits themselves stay unrounded (this engine keeps them in float32)."""
    w = W["model.embed_tokens.weight"] if c["tie"] or "lm_head.weight" not in W else W["lm_head.weight"]
    return held(rms_norm(x, W["model.norm.weight"], c["eps"])) @ w.T


def forward(cfg, W, tokens, held=_same):
    """Logits (T, V) float64 at every position of one whole sequence.  src/mashbox/gguf/archs/dense.py:309-392.
    held: see block()."""
    c = sizes(cfg)
    W = {k: v.to(F64) for k, v in W.items()}
    tokens = [int(t) for t in tokens]
    positions = np.arange(len(tokens))
    freqs = rope_frequencies(c["theta"], c["HD"], c["scaling"])
    x = W["model.embed_tokens.weight"][torch.tensor(tokens)]           # dense.py:328
    for l in range(c["L"]):
        x = block(x, W, l, c, freqs, positions, held)
    return head(x, W, c, held)


def greedy(cfg, W, prompt, n):
    """n greedy tokens after prompt, recomputing the whole sequence each time; argmax takes the lowest index of the
    maximum (src/mashbox/gguf/archs/dense.py:391)."""
    ids = list(prompt)
    out = []
    for _ in range(n):
        lg = forward(cfg, W, ids)[-1]
        t = int(torch.argmax(lg))
        out.append(t)
        ids.append(t)
    return out
