"""The Llama-3 dense decoder as data: which parts each layer has, in which order layers run, which tensors exist
under which names, and how stored names map to the engine's canonical names.

Canonical names are the GGUF names mashbox-labs/mashbox's dense module reads (src/mashbox/gguf/archs/dense.py:135-139,
241-248): token_embd, output_norm, output, rope_freqs, blk.N.attn_{norm,q,k,v,output}, blk.N.ffn_{norm,gate,up,down}.
A file may use those names directly (q/k rows already in adjacent-pair order, rope_freqs.weight as a tensor) or the
Hugging Face names (src/mashbox/hf/adapter.py:183-220), in which case q/k rows (and biases) are permuted at load so that
the rotation acts on adjacent pairs (adapter.py:223-225, 286-293).
"""
import re

from ..config.llama import LlamaConfig
from ..parts.base import LayerRun, LayerSpec, ModelSpec, PartSpec

HF_LAYER = {"self_attn.q_proj": "attn_q", "self_attn.k_proj": "attn_k", "self_attn.v_proj": "attn_v",
            "self_attn.o_proj": "attn_output", "mlp.gate_proj": "ffn_gate", "mlp.up_proj": "ffn_up",
            "mlp.down_proj": "ffn_down", "input_layernorm": "attn_norm", "post_attention_layernorm": "ffn_norm"}
HF_GLOBAL = {"embed_tokens.weight": "token_embd.weight", "norm.weight": "output_norm.weight"}
HF_PREFIXES = ("model.language_model.", "language_model.model.", "model.")
GGUF_LAYER = set(HF_LAYER.values())
GGUF_GLOBAL = {"token_embd.weight", "output_norm.weight", "output.weight", "rope_freqs.weight"}
_BLK = re.compile(r"^blk\.(\d+)\.([a-z_]+)\.(weight|bias)$")


def model_spec(c: LlamaConfig) -> ModelSpec:
    s = c.rope_scaling
    scaling = None
    if s is not None:
        scaling = ("linear", s.factor) if s.kind == "linear" else (
            "llama3", s.factor, s.low_freq_factor, s.high_freq_factor, s.original_max_position)
    rope = PartSpec("rope", head_dim=c.head_dim, rotary_dim=c.head_dim, theta=c.rope_theta, scaling=scaling,
                    pairing="adjacent", factors_name="rope_freqs.weight")
    norm = PartSpec("rms", width=c.hidden, eps=c.rms_eps)
    mixer = PartSpec("attention", hidden=c.hidden, heads=c.num_heads, kv_heads=c.num_kv_heads, head_dim=c.head_dim,
                     bias=c.attention_bias, position=rope)
    ffn = PartSpec("swiglu", hidden=c.hidden, intermediate=c.intermediate)
    layers = [LayerSpec(prefix=f"blk.{i}.", block=PartSpec("prenorm", norm=norm, mixer=mixer, ffn=ffn))
              for i in range(c.num_layers)]
    return ModelSpec(hidden=c.hidden, vocab=c.vocab,
                     embedding=PartSpec("table", vocab=c.vocab, hidden=c.hidden),
                     layers=layers, schedule=[LayerRun(layer=i, cache=i, write=True) for i in range(c.num_layers)],
                     final_norm=PartSpec("rms", width=c.hidden, eps=c.rms_eps, name="output_norm.weight"),
                     head=PartSpec("linear", vocab=c.vocab, hidden=c.hidden, tied=c.tie_embeddings))


def permute_rows(t, heads):
    """rows (heads, 2, HD/2) -> (heads, HD/2, 2): half-split rotation order to adjacent-pair order"""
    shape = t.shape
    return t.reshape((heads, 2, shape[0] // heads // 2) + tuple(shape[1:])).transpose(1, 2).reshape(shape)


def canonical_names(c: LlamaConfig):
    """-> function stored name -> (canonical name, transform or None) | None to skip; KeyError for an unknown name"""
    def canonical(name):
        if name.endswith("rotary_emb.inv_freq"):
            return None
        if name == "lm_head.weight":
            return None if c.tie_embeddings else ("output.weight", None)
        if name in GGUF_GLOBAL:
            if name == "output.weight" and c.tie_embeddings:
                return None
            return name, None
        m = _BLK.match(name)
        if m and m.group(2) in GGUF_LAYER:
            return name, None
        for p in HF_PREFIXES:
            if name.startswith(p):
                rest = name[len(p):]
                if rest in HF_GLOBAL:
                    return HF_GLOBAL[rest], None
                parts = rest.split(".")
                if len(parts) >= 4 and parts[0] == "layers" and parts[1].isdigit() and parts[-1] in ("weight", "bias"):
                    role = ".".join(parts[2:-1])
                    if role in HF_LAYER:
                        g = HF_LAYER[role]
                        transform = None
                        if g == "attn_q":
                            transform = lambda t: permute_rows(t, c.num_heads)
                        elif g == "attn_k":
                            transform = lambda t: permute_rows(t, c.num_kv_heads)
                        return f"blk.{parts[1]}.{g}.{parts[-1]}", transform
                break
        raise KeyError(name)
    return canonical


def stored_tensors(c: LlamaConfig):
    """Hugging Face names, shapes and kinds of the tensors a checkpoint of this configuration holds."""
    D, H, KV, HD, F, V = c.hidden, c.num_heads, c.num_kv_heads, c.head_dim, c.intermediate, c.vocab
    out = {"model.embed_tokens.weight": ((V, D), "matrix")}
    for i in range(c.num_layers):
        p = f"model.layers.{i}."
        out[p + "input_layernorm.weight"] = ((D,), "norm")
        for n, rows in (("q", H * HD), ("k", KV * HD), ("v", KV * HD)):
            out[p + f"self_attn.{n}_proj.weight"] = ((rows, D), "matrix")
            if c.attention_bias:
                out[p + f"self_attn.{n}_proj.bias"] = ((rows,), "bias")
        out[p + "self_attn.o_proj.weight"] = ((D, H * HD), "matrix")
        if c.attention_bias:
            out[p + "self_attn.o_proj.bias"] = ((D,), "bias")
        out[p + "post_attention_layernorm.weight"] = ((D,), "norm")
        out[p + "mlp.gate_proj.weight"] = ((F, D), "matrix")
        out[p + "mlp.up_proj.weight"] = ((F, D), "matrix")
        out[p + "mlp.down_proj.weight"] = ((D, F), "matrix")
    out["model.norm.weight"] = ((D,), "norm")
    if not c.tie_embeddings:
        out["lm_head.weight"] = ((V, D), "matrix")
    return out
