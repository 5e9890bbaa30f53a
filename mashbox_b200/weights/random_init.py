"""Random-weights mode: a model's tensors from a configuration and a seed, and a model folder written from them.

Every tensor has its own generator, seeded from (seed, crc32 of the tensor's name), so a tensor's values depend on
neither the order tensors are made in nor on which other tensors exist.  Matrices are N(0, std), norm weights
1 + N(0, norm_std), biases N(0, std).  The architecture entry says which tensors a configuration has (Hugging Face
names and shapes); nothing here knows a model.
"""
import json
import os
import zlib

import torch

from .safetensors_io import TensorSource, write_safetensors


def tensor_seed(seed, name):
    return (int(seed) * 1_000_003 + zlib.crc32(name.encode())) % (1 << 63)


def random_tensors(shapes, seed, dtype=torch.float32, device="cpu", std=0.02, norm_std=0.01, std_by_name=()):
    """shapes: {name: (shape, kind)} with kind "matrix" | "norm" | "bias" -> {name: tensor of dtype on device}.
    std_by_name: (substring, std) pairs; the first whose substring is in a matrix's or bias's name replaces std."""
    out = {}
    for name, (shape, kind) in shapes.items():
        g = torch.Generator(device=device)
        g.manual_seed(tensor_seed(seed, name))
        x = torch.randn(tuple(shape), generator=g, device=device, dtype=torch.float32)
        if kind == "norm":
            x = 1.0 + norm_std * x
        else:
            x = next((s for sub, s in std_by_name if sub in name), std) * x
        out[name] = x.to(dtype)
    return out


class RandomSource(TensorSource):
    """Seeded random tensors made when asked for, on `device` (a benchmark of a large shape makes its weights on the
    GPU and never writes them to disk).  Values depend on the device kind: a CUDA generator and a CPU generator give
    different numbers for one seed."""

    def __init__(self, shapes, seed, dtype=torch.bfloat16, device="cpu", std=0.02, norm_std=0.01, std_by_name=()):
        self.shapes, self.seed, self.dtype, self.device = dict(shapes), seed, dtype, device
        self.kw = dict(std=std, norm_std=norm_std, std_by_name=std_by_name)

    def names(self):
        return list(self.shapes)

    def info(self, name):
        return self.dtype, tuple(self.shapes[name][0])

    def get(self, name):
        return random_tensors({name: self.shapes[name]}, self.seed, self.dtype, self.device, **self.kw)[name]


def write_model_folder(folder, config, seed, dtype=torch.float32, std=0.02, norm_std=0.01, std_by_name=()):
    """Writes folder/config.json and folder/model.safetensors for `config` (an architecture's typed configuration)
    with seeded random weights stored as `dtype`.  -> folder"""
    from ..config.registry import architecture
    entry = architecture(config.architecture)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as fh:
        json.dump(config.to_hf(), fh, indent=1)
    tensors = random_tensors(entry.stored_tensors(config), seed, dtype=dtype, std=std, norm_std=norm_std,
                             std_by_name=std_by_name)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    return folder
