"""Parts a decoder is assembled from; importing this package registers the built-in ones."""
from .base import (Block, BuildEnv, CacheNeed, Deferred, FeedForward, KVNeed, LayerCache, LayerRun, Mixer, ModelSpec,
                   Norm, Part, PartError, PartSpec, PositionEncoding, WeightSpec, Workspace,
                   build, register, registered)
from . import norm, rope, attention, mlp, block  # noqa: F401  (registration)

__all__ = ["Block", "BuildEnv", "CacheNeed", "Deferred", "FeedForward", "KVNeed", "LayerCache", "LayerRun", "Mixer",
           "ModelSpec", "Norm", "Part", "PartError", "PartSpec", "PositionEncoding",
           "WeightSpec", "Workspace", "build", "register", "registered"]
