from .registry import (Architecture, known_architectures, load_config, register_architecture,
                       resolve)
from .decoder import DecoderModel
from . import llama  # noqa: F401  (registration)

__all__ = ["Architecture", "DecoderModel", "known_architectures", "load_config",
           "register_architecture", "resolve"]
