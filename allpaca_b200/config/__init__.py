from .model_config import ConfigError, LlamaConfig, RopeScaling, read_config_json
from .engine_config import EngineConfig

__all__ = ["ConfigError", "LlamaConfig", "RopeScaling", "read_config_json", "EngineConfig"]
