"""Exceptions the engine raises for a person to read: one line each, naming the field, tensor or option."""


class MashboxError(Exception):
    """Base class: a model folder, request or option this engine cannot run."""


class ConfigError(MashboxError):
    """config.json names something unsupported or leaves out a required key."""


class WeightError(MashboxError):
    """The weight files do not fit the model: missing, unexpected or wrongly shaped tensors, bad files."""


class KernelError(MashboxError):
    """The CUDA extension is missing, failed to build, or refused the sizes it was given."""


class CacheError(MashboxError):
    """The cache manager was asked for something it cannot give (no pages, unknown request)."""


class RequestError(MashboxError):
    """A request the engine refuses alone (bad ids, over the context, bad sampling settings)."""
