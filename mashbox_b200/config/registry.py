"""The one registry from an architecture's name (config.json `architectures[0]`) to its model.

An entry holds: the typed configuration class (from_hf / to_hf), model_spec(config) -> ModelSpec (the layers as data),
canonical_names(config) -> the function that maps stored tensor names to canonical ones, and stored_tensors(config) ->
the tensors a checkpoint holds (for random weights).  mashbox-labs/mashbox keeps the same kind of table
(src/mashbox/hf/adapter.py:25-29 maps LlamaForCausalLM and MistralForCausalLM to its llama module).
"""
from dataclasses import dataclass
from typing import Callable

from ..errors import ConfigError


@dataclass
class Architecture:
    name: str
    config_class: type
    model_spec: Callable
    canonical_names: Callable
    stored_tensors: Callable


ARCHITECTURES = {}


def register_architecture(entry: Architecture):
    ARCHITECTURES[entry.name] = entry
    return entry


def architecture(name) -> Architecture:
    _builtin()
    if name not in ARCHITECTURES:
        raise ConfigError(f'config.json architectures "{name}" is not read by this engine (it reads '
                          f"{', '.join(sorted(ARCHITECTURES))})")
    return ARCHITECTURES[name]


def read_config(cfg: dict):
    """config.json as a dict -> (Architecture, typed configuration)"""
    archs = cfg.get("architectures") or []
    if not archs:
        raise ConfigError("config.json has no `architectures` entry")
    entry = architecture(archs[0])
    return entry, entry.config_class.from_hf(cfg)


_done = False


def _builtin():
    global _done
    if _done:
        return
    _done = True
    from ..models import llama
    from .llama import LlamaConfig
    for name in ("LlamaForCausalLM", "MistralForCausalLM"):
        if name not in ARCHITECTURES:
            register_architecture(Architecture(name, LlamaConfig, llama.model_spec, llama.canonical_names,
                                               llama.stored_tensors))
