"""Loads the tensors a model asks for, by name, and says in one error everything that does not fit.

A model (through its architecture entry) hands the loader a list of `Want`s -- canonical name, shape, role -- and a
function from a stored name to (canonical name, transform) or None for a tensor that is knowingly not read.  The
loader checks the whole file table first: tensors the model wants and the files lack (missing), tensors of the files
with no place in the model (unexpected), and shapes that differ (wrong shape) come out in ONE WeightError.  Only then
is anything read.

dtype policy: role "matrix" (an operand of a contraction, the embedding table included) is held in the compute dtype
(bfloat16 to serve, float32 on the 32-bit path; bf16 -> f32 is exact); role "vector" (norm weights, biases, other
small per-channel values) is held in float32 whatever the file stores, as the reference does (src/mashbox/gguf/archs/
dense.py:173-177); role "table" (integer tables) is held as int32; role "keep" stays as stored.
"""
from dataclasses import dataclass
from typing import Callable, Optional

import torch

from ..errors import WeightError
from .safetensors_io import TensorSource


@dataclass(frozen=True)
class Want:
    name: str                    # canonical name
    shape: tuple
    role: str = "matrix"         # matrix | vector | table | keep
    optional: bool = False


def held_dtype(role, stored, compute):
    if role == "matrix":
        return compute
    if role == "vector":
        return torch.float32
    if role == "table":
        return torch.int32
    return stored


def load_tensors(source: TensorSource, wants, canonical: Callable, compute_dtype, device="cpu", log=None):
    """-> {canonical name: tensor on device}.  `canonical(stored name)` -> (name, transform or None), or None to
    skip the tensor; it raises KeyError for a name it does not know."""
    wanted = {w.name: w for w in wants}
    found, unexpected = {}, []
    for stored in source.names():
        try:
            m = canonical(stored)
        except KeyError:
            unexpected.append(stored)
            continue
        if m is None:
            continue
        name, transform = m
        if name not in wanted:
            unexpected.append(stored)
            continue
        if name in found:
            unexpected.append(f"{stored} (a second tensor for {name})")
            continue
        found[name] = (stored, transform)
    missing = [w.name for w in wants if not w.optional and w.name not in found]
    wrong = []
    for name, (stored, _) in found.items():
        _, shape = source.info(stored)
        if tuple(shape) != tuple(wanted[name].shape):
            wrong.append(f"{stored} is {list(shape)}, the configuration says {list(wanted[name].shape)}")
    if missing or unexpected or wrong:
        parts = []
        if missing:
            parts.append("missing: " + ", ".join(sorted(missing)))
        if unexpected:
            parts.append("unexpected: " + ", ".join(sorted(unexpected)))
        if wrong:
            parts.append("wrong shape: " + "; ".join(sorted(wrong)))
        raise WeightError("the weights do not fit the model -- " + " | ".join(parts))
    out = {}
    for name, (stored, transform) in found.items():
        t = source.get(stored)
        role = wanted[name].role
        if not t.dtype.is_floating_point and role != "table" and role != "keep":
            raise WeightError(f"tensor {stored} is stored as {t.dtype}, a {role} needs floating point values")
        if transform is not None:
            t = transform(t)
        out[name] = t.to(device=device, dtype=held_dtype(role, t.dtype, compute_dtype)).contiguous()
    if log:
        log(dict(event="weights", tensors=len(out), bytes=sum(t.numel() * t.element_size() for t in out.values())))
    return out
