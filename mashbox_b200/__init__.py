"""mashbox_b200: a small, whole inference engine for the Llama-3 dense decoder on one NVIDIA B200.

Model folder (config.json + safetensors) -> typed configuration -> layers put together from parts -> paged cache ->
one step function over mixed batches -> scheduler, sampler, command line, trace replay.  Kernels are hand-written
CUDA for sm_100a (mashbox_b200/csrc), built at first use.
"""
__version__ = "0.1.0"

from .errors import (MashboxError, ConfigError, WeightError, KernelError, CacheError, RequestError)  # noqa: F401


def Engine(*args, **kwargs):
    from .engine.engine import Engine as _Engine
    return _Engine(*args, **kwargs)


def from_folder(folder, **kwargs):
    """Engine for a model folder: from_folder(dir, dtype="bfloat16", max_tokens=65536, ...)."""
    from .engine.engine import Engine as _Engine
    return _Engine.from_folder(folder, **kwargs)
