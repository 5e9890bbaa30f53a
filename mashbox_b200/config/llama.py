"""Typed configuration of the Llama-3 dense decoder, read from config.json's own keys.

Keys, defaults and refusals follow mashbox-labs/mashbox's Hugging Face path (src/mashbox/hf/adapter.py:62-159):
KV heads default to the head count, head_dim to hidden/heads, rms_norm_eps to 1e-6, theta and scaling come from
`rope_parameters` (transformers 5) or `rope_theta` + `rope_scaling`; hidden_act other than silu, quantization_config,
mlp_bias, sliding windows, non-full layer_types, routed-expert fields and unknown rope types are refused in one line.
No size or constant of the model is written anywhere else in the package.
"""
from dataclasses import dataclass, field
from typing import Optional

from ..errors import ConfigError

MOE_FIELDS = ("num_experts", "num_local_experts", "n_routed_experts", "moe_intermediate_size")


@dataclass(frozen=True)
class RopeScaling:
    """kind: "linear" (angles x 1/factor) or "llama3" (per-pair divisors from the four numbers)."""
    kind: str
    factor: float
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position: int = 8192


@dataclass(frozen=True)
class LlamaConfig:
    architecture: str
    num_layers: int
    hidden: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    intermediate: int
    vocab: int
    rms_eps: float
    rope_theta: float
    rope_scaling: Optional[RopeScaling]
    tie_embeddings: bool
    attention_bias: bool
    max_position: int
    extra: dict = field(default_factory=dict, compare=False, hash=False)

    # ------------------------------------------------------------------------------------------ reading
    @classmethod
    def from_hf(cls, cfg: dict) -> "LlamaConfig":
        archs = cfg.get("architectures") or []
        if not archs:
            raise ConfigError("config.json has no `architectures` entry")
        arch = archs[0]

        def need(key):
            if cfg.get(key) is None:
                raise ConfigError(f"config.json has no `{key}`")
            return cfg[key]

        def no(key, value):
            return ConfigError(f"config.json {key} = {value!r} is not supported for {arch}")

        act = cfg.get("hidden_act", cfg.get("hidden_activation", "silu"))
        if act != "silu":
            raise no("hidden_act", act)
        if cfg.get("quantization_config"):
            raise no("quantization_config", cfg["quantization_config"].get("quant_method", "set"))
        if cfg.get("mlp_bias"):
            raise no("mlp_bias", True)
        if cfg.get("use_sliding_window"):
            raise no("use_sliding_window", True)
        if cfg.get("sliding_window"):
            raise no("sliding_window", cfg["sliding_window"])
        kinds = cfg.get("layer_types") or []
        if any(k != "full_attention" for k in kinds):
            raise no("layer_types", sorted(set(kinds)))
        for key in MOE_FIELDS:
            if cfg.get(key):
                raise no(key, cfg[key])
        heads = int(need("num_attention_heads"))
        hidden = int(need("hidden_size"))
        kv = int(cfg.get("num_key_value_heads") or heads)
        head_dim = int(cfg.get("head_dim") or hidden // heads)
        if heads % kv:
            raise no("num_key_value_heads", kv)
        if head_dim % 2:
            raise no("head_dim", head_dim)
        rp = cfg.get("rope_parameters") or {}
        theta = float(rp.get("rope_theta", cfg.get("rope_theta", 10000.0)))
        sc = cfg.get("rope_scaling") or None
        if rp.get("rope_type") not in (None, "default"):
            sc = rp
        kind = (sc or {}).get("rope_type", (sc or {}).get("type"))
        if kind in (None, "default"):
            scaling = None
        elif kind == "linear":
            scaling = RopeScaling("linear", float(sc["factor"]))
        elif kind == "llama3":
            scaling = RopeScaling("llama3", float(sc.get("factor", 8.0)), float(sc.get("low_freq_factor", 1.0)),
                                  float(sc.get("high_freq_factor", 4.0)),
                                  int(sc.get("original_max_position_embeddings", 8192)))
        else:
            raise no("rope type", kind)
        return cls(architecture=arch, num_layers=int(need("num_hidden_layers")), hidden=hidden, num_heads=heads,
                   num_kv_heads=kv, head_dim=head_dim, intermediate=int(need("intermediate_size")),
                   vocab=int(need("vocab_size")), rms_eps=float(cfg.get("rms_norm_eps", 1e-6)), rope_theta=theta,
                   rope_scaling=scaling, tie_embeddings=bool(cfg.get("tie_word_embeddings", False)),
                   attention_bias=bool(cfg.get("attention_bias", False)),
                   max_position=int(cfg.get("max_position_embeddings") or 0),
                   extra={k: cfg[k] for k in ("bos_token_id", "eos_token_id") if k in cfg})

    # ------------------------------------------------------------------------------------------ writing
    def to_hf(self) -> dict:
        """The config.json that `from_hf` reads back to this configuration (random-weights mode writes it)."""
        out = {"architectures": [self.architecture], "model_type": "llama", "hidden_act": "silu",
               "num_hidden_layers": self.num_layers, "hidden_size": self.hidden,
               "num_attention_heads": self.num_heads, "num_key_value_heads": self.num_kv_heads,
               "head_dim": self.head_dim, "intermediate_size": self.intermediate, "vocab_size": self.vocab,
               "rms_norm_eps": self.rms_eps, "rope_theta": self.rope_theta,
               "tie_word_embeddings": self.tie_embeddings, "attention_bias": self.attention_bias,
               "max_position_embeddings": self.max_position}
        s = self.rope_scaling
        if s is not None and s.kind == "linear":
            out["rope_scaling"] = {"rope_type": "linear", "factor": s.factor}
        elif s is not None:
            out["rope_scaling"] = {"rope_type": "llama3", "factor": s.factor, "low_freq_factor": s.low_freq_factor,
                                   "high_freq_factor": s.high_freq_factor,
                                   "original_max_position_embeddings": s.original_max_position}
        out.update(self.extra)
        return out
