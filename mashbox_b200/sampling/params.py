"""Sampling settings of one request, with the names, defaults and checks of mashbox-labs/mashbox's sampler
(src/mashbox/runtime/sampler.py:18-67): temperature 0 = greedy, top_k 0 = off, top_p 1.0 = off, min_p 0 = off,
repetition_penalty 1.0, frequency_penalty 0, presence_penalty 0, seed 0 (64-bit)."""
import math
from dataclasses import dataclass

import numpy as np

I32_MAX = 2 ** 31 - 1


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    seed: int = 0

    @property
    def greedy(self):
        return self.temperature <= 0.0

    @property
    def penalised(self):
        return self.repetition_penalty != 1.0 or self.frequency_penalty != 0.0 or self.presence_penalty != 0.0

    @property
    def plain_greedy(self):
        return self.greedy and not self.penalised


def check_settings(r, vocab):
    """None when the settings dict r (None = greedy) fits, else the reason in one line."""
    if not r:
        return None
    if isinstance(r, SamplingParams):
        r = r.__dict__
    if not isinstance(r, dict):
        return "sampling settings must be an object"
    try:
        f = {n: float(d if r.get(n) is None else r[n]) for n, d in (
            ("temperature", 0.0), ("top_p", 1.0), ("min_p", 0.0), ("repetition_penalty", 1.0),
            ("frequency_penalty", 0.0), ("presence_penalty", 0.0))}
        k = r.get("top_k") or 0
        seed = r.get("seed") or 0
    except (TypeError, ValueError, OverflowError):
        return "sampling settings must be numbers"
    if not all(math.isfinite(v) for v in f.values()):
        return "sampling settings must be finite numbers"
    if isinstance(k, bool) or not isinstance(k, (int, np.integer)) or not 0 <= int(k) <= vocab:
        return f"top_k must be an integer 0..{vocab} (the vocabulary size)"
    if isinstance(seed, bool) or not isinstance(seed, (int, np.integer)) or not -(1 << 63) <= int(seed) < (1 << 64):
        return "seed must be an integer that fits 64 bits"
    if not (f["temperature"] >= 0 and 0 < f["top_p"] <= 1 and 0 <= f["min_p"] < 1 and f["repetition_penalty"] > 0):
        return "temperature >= 0, top_p (0, 1], min_p [0, 1), repetition_penalty > 0"
    return None


def make_params(r):
    """dict | SamplingParams | None -> SamplingParams (call check_settings first)"""
    if r is None:
        return SamplingParams()
    if isinstance(r, SamplingParams):
        return r
    g = lambda n, d: d if r.get(n) is None else r[n]
    return SamplingParams(temperature=float(g("temperature", 0.0)), top_k=int(r.get("top_k") or 0),
                          top_p=float(g("top_p", 1.0)), min_p=float(g("min_p", 0.0)),
                          repetition_penalty=float(g("repetition_penalty", 1.0)),
                          frequency_penalty=float(g("frequency_penalty", 0.0)),
                          presence_penalty=float(g("presence_penalty", 0.0)),
                          seed=int(r.get("seed") or 0) & ((1 << 64) - 1))
