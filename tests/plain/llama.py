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


def rope_frequencies(theta, rd, scaling, stored=None):
    """float32 angle per position step for each rotated pair: inv_i = theta^(-2i/RD) (src/mashbox/gguf/archs/
    dense.py:302), divided by the file's rope_freqs.weight when it has one, else by the llama3 factors when the
    configuration asks for them (dense.py:316; the Hugging Face path makes that tensor from the configuration,
    src/mashbox/hf/adapter.py:263-265), times 1/factor for linear scaling (dense.py:93-94, 317)."""
    inv = (1.0 / (np.float32(theta) ** (np.arange(0, rd, 2, dtype=np.int64).astype(np.float32) / np.float32(rd)))
           ).astype(np.float32)
    kind = (scaling or {}).get("rope_type", (scaling or {}).get("type"))
    if kind not in (None, "default", "linear", "llama3"):
        raise ValueError(kind)
    if stored is not None:
        inv = (inv / np.asarray(stored, np.float32)).astype(np.float32)
    elif kind == "llama3":
        inv = (inv / llama3_factors(theta, rd, scaling)).astype(np.float32)
    if kind == "linear":
        inv = (inv * np.float32(1.0 / float(scaling["factor"]))).astype(np.float32)
    return inv


def rope_adjacent(x, positions, freqs):
    """Rotate adjacent pairs (x[2i], x[2i+1]) by angle pos * freq_i; dims past 2*len(freqs) pass through.
    src/mashbox/gguf/archs/dense.py:280-290 (NORM form), angles dense.py:317-318 (float32 product).
    x (T, heads, HD), positions (T,) ints."""
    rd = 2 * len(freqs)
    ang = (np.asarray(positions, np.float32)[:, None] * np.asarray(freqs, np.float32)[None, :]).astype(np.float32)
    ang = torch.from_numpy(ang.astype(np.float64)).to(x.device)
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., 0:rd:2], x[..., 1:rd:2]
    rot = torch.stack([a * cos - b * sin, a * sin + b * cos], -1).reshape(x.shape[:-1] + (rd,))
    return torch.cat([rot, x[..., rd:]], -1)


def rope_halves(x, positions, freqs):
    """Rotate (x[i], x[i + RD/2]) -- the NEOX form of src/mashbox/gguf/archs/dense.py:284-286; equal to the
    adjacent form on permuted rows (that equality is what the permutation is for)."""
    rd = 2 * len(freqs)
    ang = (np.asarray(positions, np.float32)[:, None] * np.asarray(freqs, np.float32)[None, :]).astype(np.float32)
    ang = torch.from_numpy(ang.astype(np.float64)).to(x.device)
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
    pos = (torch.arange(T) if positions is None else torch.as_tensor(positions)).to(q.device)
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


# Tensor names of a layer and of the model in the two conventions a file may use: Hugging Face
# (src/mashbox/hf/adapter.py:183-192) and GGUF (src/mashbox/gguf/archs/dense.py:135-139, 241-248).
HF_NAMES = dict(layer="model.layers.{}.", ln1="input_layernorm", q="self_attn.q_proj", k="self_attn.k_proj",
                v="self_attn.v_proj", o="self_attn.o_proj", ln2="post_attention_layernorm", gate="mlp.gate_proj",
                up="mlp.up_proj", down="mlp.down_proj", embed="model.embed_tokens.weight", norm="model.norm.weight",
                head="lm_head.weight", permute=True)
GGUF_NAMES = dict(layer="blk.{}.", ln1="attn_norm", q="attn_q", k="attn_k", v="attn_v", o="attn_output",
                  ln2="ffn_norm", gate="ffn_gate", up="ffn_up", down="ffn_down", embed="token_embd.weight",
                  norm="output_norm.weight", head="output.weight", permute=False)


def block(x, W, l, c, freqs, positions, held=_same, names=HF_NAMES):
    """One pre-norm residual block: x += attn(ln1(x)); x += ffn(ln2(x)).  src/mashbox/gguf/archs/dense.py:339-357.
    With Hugging Face names q/k rows are permuted here as the loader of the reference does; GGUF-named q/k rows are
    in adjacent-pair order already (src/mashbox/hf/adapter.py:223-225 is what a converter did to them).  `held` is
    applied to every tensor the reference holds in its activation dtype (dense.py:335-357: the results of rms, of
    every matmul, of the rotation and of silu*up are cast to `act`; biases are added in float32 before the cast of q,
    k, v and after it for the output); the identity gives the exact model, round_bf16 a model of bfloat16 storage."""
    p = names["layer"].format(l)
    T = x.shape[0]
    H, KV, HD = c["H"], c["KV"], c["HD"]
    weight = lambda n: W[p + names[n] + ".weight"]
    bias = lambda n: W.get(p + names[n] + ".bias")
    plus = lambda y, b: y if b is None else y + b
    h = held(rms_norm(x, weight("ln1"), c["eps"]))
    wq, wk, bq, bk = weight("q"), weight("k"), bias("q"), bias("k")
    if names["permute"]:
        wq, wk = permute_rows(wq, H), permute_rows(wk, KV)
        bq = None if bq is None else permute_rows(bq, H)
        bk = None if bk is None else permute_rows(bk, KV)
    q = plus(held(linear(h, wq)), bq).reshape(T, H, HD)
    k = plus(held(linear(h, wk)), bk).reshape(T, KV, HD)
    v = held(plus(held(linear(h, weight("v"))), bias("v"))).reshape(T, KV, HD)
    q, k = held(rope_adjacent(q, positions, freqs)), held(rope_adjacent(k, positions, freqs))
    o = held(attention(q, k, v, HD ** -0.5, window=c.get("window"), positions=positions))
    x = x + plus(held(linear(o, weight("o"))), bias("o"))
    h = held(rms_norm(x, weight("ln2"), c["eps"]))
    g = held(linear(h, weight("gate")))
    u = held(linear(h, weight("up")))
    a = held(g * torch.sigmoid(g) * u)                                  # dense.py:356
    return x + held(linear(a, weight("down")))


def head(x, W, c, held=_same, names=HF_NAMES):
    """logits = rms(x, norm) W_head^T; the head is the embedding when tied.  src/mashbox/gguf/archs/dense.py:386-390,
    tie dense.py:129.  The logits themselves stay unrounded (this engine keeps them in float32)."""
    w = W[names["embed"]] if c["tie"] or names["head"] not in W else W[names["head"]]
    return held(rms_norm(x, W[names["norm"]], c["eps"])) @ w.T


def forward(cfg, W, tokens, held=_same, device=None, rows=None):
    """Logits (T, V) float64 at every position of one whole sequence (rows: only at these positions).
    src/mashbox/gguf/archs/dense.py:309-392.  held: see block().  The tensors may carry Hugging Face names or GGUF
    names (told apart by the embedding's name); a GGUF-named set may bring rope_freqs.weight.  device: where the
    float64 arithmetic runs (a large model is slow on the CPU)."""
    c = sizes(cfg)
    names = GGUF_NAMES if GGUF_NAMES["embed"] in W else HF_NAMES
    W = {k: torch.as_tensor(v).to(device=device, dtype=F64) for k, v in W.items()}
    tokens = [int(t) for t in tokens]
    positions = np.arange(len(tokens))
    stored = W["rope_freqs.weight"].cpu().numpy() if "rope_freqs.weight" in W else None
    freqs = rope_frequencies(c["theta"], c["HD"], c["scaling"], stored)
    x = W[names["embed"]][torch.tensor(tokens, device=device)]          # dense.py:328
    for l in range(c["L"]):
        x = block(x, W, l, c, freqs, positions, held, names)
    if rows is not None:
        x = x[torch.as_tensor(list(rows), device=device)]
    return head(x, W, c, held, names)


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
