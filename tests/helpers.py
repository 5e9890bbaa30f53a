"""Tiny configurations and shared plumbing of the tests.  Model folders are made in temporary folders."""
import functools
import json
import os

import numpy as np
import torch

from mashbox_b200.config.llama import LlamaConfig, RopeScaling
from mashbox_b200.weights.random_init import write_model_folder
from tests.plain import llama as plain

# two tiny configurations that differ in every size and option
TINY_A = LlamaConfig(architecture="LlamaForCausalLM", num_layers=2, hidden=64, num_heads=4, num_kv_heads=2, head_dim=16,
                     intermediate=192, vocab=256, rms_eps=1e-5, rope_theta=10000.0, rope_scaling=None,
                     tie_embeddings=True, attention_bias=False, max_position=256)
TINY_B = LlamaConfig(architecture="LlamaForCausalLM", num_layers=3, hidden=96, num_heads=6, num_kv_heads=1, head_dim=32,
                     intermediate=320, vocab=509, rms_eps=1e-6, rope_theta=500000.0,
                     rope_scaling=RopeScaling("llama3", 8.0, 1.0, 4.0, 64), tie_embeddings=False, attention_bias=True,
                     max_position=512)
# a third one with the head size of the large models, so that the engine-level tests reach the kernels that take only
# head size 128 (the tcgen05 attention kernel) and 64/128 (the TMA-fed one): linear rope scaling, 2 query heads per kv head
TINY_C = LlamaConfig(architecture="LlamaForCausalLM", num_layers=2, hidden=256, num_heads=4, num_kv_heads=2, head_dim=128,
                     intermediate=384, vocab=311, rms_eps=1e-5, rope_theta=1000000.0,
                     rope_scaling=RopeScaling("linear", 2.0), tie_embeddings=False, attention_bias=False,
                     max_position=1024)
# and a fourth with heads of 64 (not hidden / heads), three query heads per kv head, biases and a tied head: the head
# size of the smallest models, which the TMA-fed and tcgen05 attention kernels take in a form of its own
TINY_D = LlamaConfig(architecture="LlamaForCausalLM", num_layers=2, hidden=192, num_heads=6, num_kv_heads=2, head_dim=64,
                     intermediate=272, vocab=401, rms_eps=1e-5, rope_theta=10000.0,
                     rope_scaling=RopeScaling("llama3", 4.0, 1.0, 4.0, 32), tie_embeddings=True, attention_bias=True,
                     max_position=1024)
TINY = {"A": (TINY_A, 0, 16), "B": (TINY_B, 1, 8), "C": (TINY_C, 2, 16), "D": (TINY_D, 3, 32)}   # config, seed, page size
# Random weights shaped like a trained model's rather than like an initialisation: an embedding of order one, readers
# (q, k, v, gate, up, head) near 1/sqrt(fan in) so that attention is not uniform, and writers into the residual stream
# (o_proj, down_proj) small, so that a layer changes the stream a little instead of replacing it.  With every matrix
# at one width the stream is whatever the last layer wrote and the model amplifies any perturbation about seven-fold
# per layer (measured: one-step bf16 differences in 1e-4 of the first product's outputs reached most values two layers
# later), which buries every comparison in bfloat16 under noise.
# Readers are N(0, STD(hidden)) with STD about 1/sqrt(fan in), so that q, k and the scores are of order one at every width
# (at 0.1 the 256-wide model C has scores of standard deviation 2.6 and a softmax sharp enough to turn one-step bf16
# differences of the first product into 1.4e-5 of the logits).
def STD(hidden):
    return min(0.1, hidden ** -0.5)


STD_BY_NAME = (("embed_tokens", 1.0), ("o_proj", 0.02), ("down_proj", 0.02))


def make_folder(tmp, name, store="float32"):
    cfg, seed, _ = TINY[name]
    d = os.path.join(str(tmp), f"tiny_{name}_{store}")
    if not os.path.isdir(d):
        write_model_folder(d, cfg, seed, dtype=getattr(torch, store), std=STD(cfg.hidden), norm_std=0.1,
                           std_by_name=STD_BY_NAME)
    return d


@functools.lru_cache(maxsize=None)
def _plain_model(folder):
    return plain.read_model(folder)


def plain_logits(folder, tokens):
    """float64 logits (T, V) of the plain implementation for one whole sequence"""
    cfg, W = _plain_model(folder)
    return plain.forward(cfg, W, tokens).numpy()


def plain_rounded(folder, tokens):
    """the same with every tensor the engine holds in bfloat16 rounded to bfloat16"""
    cfg, W = _plain_model(folder)
    return plain.forward(cfg, W, tokens, held=plain.round_bf16).numpy()


# (dtype, engine options): float32; bfloat16 with the plain attention kernel; bfloat16 with the tensor-core kernel
MODES = {"f32": ("float32", {}), "bf16-plain": ("bfloat16", {"plain_attention": True}), "bf16": ("bfloat16", {})}


def check(got, folder, tokens, mode, what, rows=slice(None)):
    from tests.tolerances import assert_logits
    dtype, options = MODES[mode]
    want = plain_logits(folder, tokens)[rows]
    rounded = plain_rounded(folder, tokens)[rows] if dtype == "bfloat16" else None
    return assert_logits(got, want, dtype, what, rounded, same_rounding=bool(options.get("plain_attention")))


def prompts_for(name, lengths, seed=0):
    cfg = TINY[name][0]
    rng = np.random.default_rng(seed)
    return [rng.integers(0, cfg.vocab, n).tolist() for n in lengths]


def store_for(dtype):
    """weights are stored in the dtype the run computes in, so the plain implementation sees the same values"""
    return "float32" if dtype == "float32" else "bfloat16"
