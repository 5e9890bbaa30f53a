"""Parts a layer is put together from.  Importing this package registers the built-in kinds."""
from . import base, norm, position, attention, feed_forward, block, embedding  # noqa: F401
from .base import (PartSpec, LayerSpec, LayerRun, ModelSpec, Env, StepContext, StepInputs, Workspace,  # noqa: F401
                   register, make)
