"""Reading and writing safetensors files by tensor name, with the standard library, NumPy and torch only.

The format: 8 bytes little-endian length of a JSON header, the header {name: {dtype, shape, data_offsets}} (an optional
"__metadata__" entry beside the tensors), then the tensors' bytes, data_offsets counting from the end of the header.
Which files of a folder hold the weights (mashbox-labs/mashbox decides the same way, src/mashbox/hf/source.py:43-55): the
shards that model.safetensors.index.json's weight_map names, else the folder's own `model.safetensors` /
`model-00001-of-0000N.safetensors` files, else every *.safetensors there is -- so a second copy of the weights under
another name (Mistral repositories ship `consolidated.safetensors` beside the shards) is not read twice.
BF16, F16, F32 and the integer types I32/I64 are read; anything else is refused by name.
"""
import json
import os
import re
import struct

import numpy as np
import torch

from ..errors import WeightError

ITEM = {"BF16": 2, "F16": 2, "F32": 4, "I32": 4, "I64": 8}
TORCH = {"BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "I32": torch.int32, "I64": torch.int64}
NAME = {v: k for k, v in TORCH.items()}
VIEW = {"BF16": np.int16, "F16": np.float16, "F32": np.float32, "I32": np.int32, "I64": np.int64}
INDEX_FILE = "model.safetensors.index.json"
MODEL_FILE = re.compile(r"^model(-\d+-of-\d+)?\.safetensors$")


def weight_files(folder):
    """-> paths of the files that hold the folder's weights (a file the index names may be absent: the caller says so)"""
    index = os.path.join(folder, INDEX_FILE)
    if os.path.isfile(index):
        with open(index) as fh:
            named = set(json.load(fh).get("weight_map", {}).values())
        return [os.path.join(folder, n) for n in sorted(named)]
    present = sorted(n for n in os.listdir(folder) if n.endswith(".safetensors")) if os.path.isdir(folder) else []
    own = [n for n in present if MODEL_FILE.match(n)]
    return [os.path.join(folder, n) for n in (own or present)]


class Shard:
    """One safetensors file: its header checked against the file's size, its tensors as (dtype name, shape, first byte,
    end byte) under their names, its bytes as a read-only memory map."""

    def __init__(self, path):
        self.path, self.label = path, os.path.basename(path)
        size = os.path.getsize(path)
        with open(path, "rb") as fh:
            prefix = fh.read(8)
            length = struct.unpack("<Q", prefix)[0] if len(prefix) == 8 else None
            if length is None or length < 2 or 8 + length > size:
                raise WeightError(f"{self.label}: no safetensors header (the file is {size} bytes"
                                  + ("" if length is None else f", its first 8 bytes announce a header of {length}") + ")")
            try:
                table = json.loads(fh.read(length))
            except ValueError as e:
                raise WeightError(f"{self.label}: the safetensors header is not JSON ({e})") from None
        if not isinstance(table, dict):
            raise WeightError(f"{self.label}: the safetensors header is not a table of tensors")
        table.pop("__metadata__", None)
        start, room = 8 + length, size - 8 - length
        self.tensors = {}
        for name, entry in table.items():
            kind = entry.get("dtype")
            if kind not in ITEM:
                raise WeightError(f"{self.label}: tensor {name} has dtype {kind}; this engine reads {', '.join(sorted(ITEM))}")
            shape = tuple(int(d) for d in entry["shape"])
            first, end = (int(v) for v in entry["data_offsets"])
            want = int(np.prod(shape, dtype=np.int64)) * ITEM[kind]
            if not 0 <= first <= end <= room or end - first != want:
                raise WeightError(f"{self.label}: tensor {name} of shape {list(shape)} and dtype {kind} needs {want} bytes, "
                                  f"its entry gives bytes {first}..{end} of {room}")
            self.tensors[name] = (kind, shape, start + first, start + end)
        self.bytes = np.memmap(path, dtype=np.uint8, mode="r")


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
        paths = weight_files(folder)
        if not paths:
            raise WeightError(f"{folder}: no safetensors weights in this folder")
        absent = [os.path.basename(p) for p in paths if not os.path.isfile(p)]
        if absent:
            raise WeightError(f"{folder}: {INDEX_FILE} names {', '.join(absent)}, which the folder does not have")
        self.shards = [Shard(p) for p in paths]
        self.where = {}
        for shard in self.shards:
            for name in shard.tensors:
                if name in self.where:
                    raise WeightError(f"{folder}: tensor {name} is in {self.where[name].label} and in {shard.label}")
                self.where[name] = shard

    def names(self):
        return list(self.where)

    def info(self, name):
        kind, shape = self.where[name].tensors[name][:2]
        return TORCH[kind], shape

    def get(self, name):
        shard = self.where[name]
        kind, shape, first, end = shard.tensors[name]
        a = np.array(shard.bytes[first:end]).view(VIEW[kind]).reshape(shape)          # one copy out of the map
        t = torch.from_numpy(a)
        return t.view(torch.bfloat16) if kind == "BF16" else t

    def close(self):
        self.shards, self.where = [], {}


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
