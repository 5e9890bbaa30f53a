"""From a model folder (config.json + safetensors) to a model with its weights bound on the device."""
import json
import os

import torch

from ..config.registry import read_config
from ..errors import ConfigError
from ..models.model import Model
from ..parts import Env
from ..weights.loader import load_tensors
from ..weights.safetensors_io import SafetensorsSource

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
          "f32": torch.float32}


def torch_dtype(name):
    if isinstance(name, torch.dtype):
        return name
    if name not in DTYPES:
        raise ConfigError(f"dtype {name!r}: bfloat16 or float32")
    return DTYPES[name]


def read_config_file(folder):
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{folder} has no config.json")
    with open(path) as fh:
        return json.load(fh)


def build_model(cfg_dict, source, dtype, device, ops=None, log=None):
    """config.json dict + a TensorSource -> Model with weights on `device` in compute dtype `dtype`."""
    entry, config = read_config(cfg_dict)
    model = Model(entry.model_spec(config), config)
    dt = torch_dtype(dtype)
    tensors = load_tensors(source, model.wants(), entry.canonical_names(config), dt, device, log=log)
    model.bind(tensors, Env(dt, device, ops))
    return model


def load_model(folder, dtype="bfloat16", device="cuda:0", log=None):
    from .. import ops
    source = SafetensorsSource(folder)
    try:
        return build_model(read_config_file(folder), source, dtype, device, ops=ops, log=log)
    finally:
        source.close()
