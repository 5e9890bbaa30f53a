"""Rotary position encoding with the Llama-3 frequency scaling.

Angle of pair i at position p: p * freq_i (a float32 product, src/mashbox/gguf/archs/dense.py:317) with
freq_i = theta^(-2i/RD) (dense.py:302), divided by the llama3 factor of the pair (dense.py:316; factors as
src/mashbox/hf/adapter.py:162-179, or the tensor rope_freqs.weight when the file brings one) or multiplied by 1/factor for
linear scaling (dense.py:93-94).  Pairs are adjacent (2i, 2i+1) -- the loader permutes Hugging Face q/k rows for that --
or halves (i, i + RD/2) (dense.py:280-290).  Dims from RD on pass through.  The rotation itself happens inside the
rotate-and-store kernel of the mixer; this part owns the frequency table.
"""
import math

import numpy as np

from ..weights.loader import Want
from .base import register

PAIRINGS = {"adjacent": 0, "halves": 1}


def llama3_factors(theta, dim, factor, low, high, original):
    """One divisor per rotated pair: wavelengths under original/high keep their frequency, over original/low are
    slowed by `factor`, between the two a smooth blend."""
    freqs = 1.0 / (np.float32(theta) ** (np.arange(0, dim, 2, dtype=np.float32) / np.float32(dim)))
    out = np.empty(len(freqs), np.float32)
    for i, f in enumerate(freqs):
        wave = 2 * math.pi / float(f)
        if wave < original / high:
            out[i] = 1.0
        elif wave > original / low:
            out[i] = factor
        else:
            s = (original / wave - low) / (high - low)
            out[i] = 1.0 / ((1 - s) / factor + s)
    return out


def base_frequencies(theta, rotary_dim):
    return (1.0 / (np.float32(theta) ** (np.arange(0, rotary_dim, 2, dtype=np.int64).astype(np.float32)
                                         / np.float32(rotary_dim)))).astype(np.float32)


class RotaryEncoding:
    graph_safe = True       # forward() depends on the batch only through the lengths of the step's arrays
    def __init__(self, head_dim, rotary_dim, theta, scaling=None, pairing="adjacent", factors_name=None):
        """scaling: None | ("linear", factor) | ("llama3", factor, low, high, original).  factors_name: canonical name
        of an optional tensor of per-pair divisors that replaces the computed llama3 factors when the file has it."""
        self.head_dim, self.rotary_dim, self.theta = int(head_dim), int(rotary_dim), float(theta)
        self.scaling = tuple(scaling) if scaling else None
        self.pairing, self.factors_name = PAIRINGS[pairing], factors_name
        self.freqs = None

    def wants(self):
        if self.factors_name is None:
            return []
        return [Want(self.factors_name, (self.rotary_dim // 2,), "vector", optional=True)]

    def frequencies(self, stored_factors=None):
        """float32 angle per position step of every rotated pair.  Stored divisors stand in for the computed llama3
        ones; the linear factor multiplies whatever the divisors are (the reference divides by the stored tensor and
        multiplies by 1/factor in the same expression, dense.py:316-317)."""
        f = base_frequencies(self.theta, self.rotary_dim)
        kind = self.scaling[0] if self.scaling else None
        if kind not in (None, "linear", "llama3"):
            raise ValueError(self.scaling)
        if stored_factors is not None:
            f = (f / np.asarray(stored_factors, np.float32)).astype(np.float32)
        elif kind == "llama3":
            _, factor, low, high, original = self.scaling
            f = (f / llama3_factors(self.theta, self.rotary_dim, factor, low, high, original)).astype(np.float32)
        if kind == "linear":
            f = (f * np.float32(1.0 / self.scaling[1])).astype(np.float32)
        return f

    def bind(self, tensors, env):
        import torch
        stored = tensors.get(self.factors_name) if self.factors_name else None
        f = self.frequencies(None if stored is None else stored.detach().float().cpu().numpy())
        self.freqs = torch.from_numpy(f).to(env.device)

    def rotation(self):
        return self.freqs, self.rotary_dim, self.pairing


register("position", "rope", RotaryEncoding)
