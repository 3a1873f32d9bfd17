from . import attention, block, embedding, feed_forward, norms, positions  # noqa: F401  (register parts)
from .base import (
    KVCacheSpec,
    Part,
    PartSpec,
    StateSpec,
    build_part,
    register_part,
    registered_parts,
)
from .context import CacheView, HostBatch, StepContext, Workspace
from .model import LayerCall, Model, ModelRecipe

__all__ = [
    "CacheView",
    "HostBatch",
    "KVCacheSpec",
    "LayerCall",
    "Model",
    "ModelRecipe",
    "Part",
    "PartSpec",
    "StateSpec",
    "StepContext",
    "Workspace",
    "build_part",
    "register_part",
    "registered_parts",
]
