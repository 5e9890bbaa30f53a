"""Reading and writing safetensors files by tensor name, with the standard library, NumPy and torch only.

Format (as mashbox-labs/mashbox reads it, src/mashbox/hf/source.py:58-101): 8 bytes little-endian header length, a
JSON header {name: {dtype, shape, data_offsets}}, then the data.  Shards come from model.safetensors.index.json's
weight_map, else every *.safetensors of the folder except Mistral's consolidated copy (source.py:21, 43-55).
BF16, F16, F32 and the integer types I32/I64 are read; anything else is refused by name.
"""
import glob
import json
import os
import struct

import numpy as np
import torch

from ..errors import WeightError

ITEM = {"BF16": 2, "F16": 2, "F32": 4, "I32": 4, "I64": 8}
TORCH = {"BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "I32": torch.int32, "I64": torch.int64}
NAME = {v: k for k, v in TORCH.items()}
VIEW = {"BF16": np.int16, "F16": np.float16, "F32": np.float32, "I32": np.int32, "I64": np.int64}
SKIP_FILES = ("consolidated.safetensors",)


def weight_files(folder):
    idx = os.path.join(folder, "model.safetensors.index.json")
    if os.path.isfile(idx):
        names = sorted(set(json.load(open(idx))["weight_map"].values()))
        return [os.path.join(folder, n) for n in names]
    return sorted(p for p in glob.glob(os.path.join(folder, "*.safetensors"))
                  if os.path.basename(p) not in SKIP_FILES)


def read_header(path):
    """-> (header dict without __metadata__, offset of the data)"""
    base = os.path.basename(path)
    with open(path, "rb") as fh:
        head = fh.read(8)
        if len(head) < 8:
            raise WeightError(f"{base} is not a safetensors file")
        (n,) = struct.unpack("<Q", head)
        if n > 100_000_000 or n + 8 > os.path.getsize(path):
            raise WeightError(f"{base} has a bad safetensors header")
        try:
            header = json.loads(fh.read(n))
        except ValueError:
            raise WeightError(f"{base} has a bad safetensors header") from None
    header.pop("__metadata__", None)
    return header, 8 + n


class TensorSource:
    """name -> tensor, with the stored dtype and shape known before anything is read."""

    def names(self):
        raise NotImplementedError

    def info(self, name):
        """-> (torch dtype, shape tuple)"""
        raise NotImplementedError

    def get(self, name) -> torch.Tensor:
        """the tensor as stored (its own dtype), on the CPU unless the source makes tensors elsewhere"""
        raise NotImplementedError

    def close(self):
        pass


class SafetensorsSource(TensorSource):
    def __init__(self, folder):
        files = weight_files(folder)
        if not files:
            raise WeightError(f"{folder} holds no *.safetensors weights")
        self.entries, self.maps = {}, []
        for p in files:
            if not os.path.isfile(p):
                raise WeightError(f"shard {os.path.basename(p)} is missing from {folder}")
            header, base = read_header(p)
            mm = np.memmap(p, dtype=np.uint8, mode="r")
            self.maps.append(mm)
            for name, t in header.items():
                dt = t["dtype"]
                if dt not in ITEM:
                    raise WeightError(f"tensor {name} is stored as {dt}; this engine reads {', '.join(sorted(ITEM))}")
                b, e = t["data_offsets"]
                shape = tuple(int(s) for s in t["shape"])
                if e - b != int(np.prod(shape, dtype=np.int64)) * ITEM[dt] or base + e > mm.shape[0]:
                    raise WeightError(f"tensor {name} in {os.path.basename(p)} has a size that does not match its shape")
                self.entries[name] = (dt, shape, mm, base + b, base + e)

    def names(self):
        return list(self.entries)

    def info(self, name):
        dt, shape = self.entries[name][:2]
        return TORCH[dt], shape

    def get(self, name):
        dt, shape, mm, b, e = self.entries[name]
        a = np.array(mm[b:e]).view(VIEW[dt]).reshape(shape)          # one copy out of the map
        t = torch.from_numpy(a)
        return t.view(torch.bfloat16) if dt == "BF16" else t

    def close(self):
        self.maps = []
        self.entries = {}


class DictSource(TensorSource):
    """Tensors already in memory, by name (tests, GGUF-named tensors read elsewhere, random weights)."""

    def __init__(self, tensors):
        self.tensors = dict(tensors)

    def names(self):
        return list(self.tensors)

    def info(self, name):
        t = self.tensors[name]
        return t.dtype, tuple(t.shape)

    def get(self, name):
        return self.tensors[name]


def write_safetensors(path, tensors):
    """tensors: {name: tensor} (any device) -> one safetensors file; data written tensor by tensor."""
    header, at = {}, 0
    for name, t in tensors.items():
        if t.dtype not in NAME:
            raise WeightError(f"tensor {name}: dtype {t.dtype} cannot be written")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": NAME[t.dtype], "shape": list(t.shape), "data_offsets": [at, at + n]}
        at += n
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * (-len(blob) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        for name, t in tensors.items():
            c = t.detach().contiguous().cpu()
            c = c.view(torch.int16) if c.dtype == torch.bfloat16 else c
            fh.write(c.numpy().tobytes())
