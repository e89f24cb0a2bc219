"""allpaca_b200: a small, whole inference engine for the dense Llama decoder on one B200.

    from allpaca_b200 import LLM, SamplingParams
    out = LLM(model="path/to/folder").generate([[1, 2, 3]], SamplingParams(max_tokens=8))
"""
from .sampling.params import SamplingParams

__version__ = "0.1.0"
__all__ = ["LLM", "SamplingParams", "RequestOutput", "EngineConfig"]


def __getattr__(name):
    if name in ("LLM", "RequestOutput"):
        from .engine import llm
        return getattr(llm, name)
    if name == "EngineConfig":
        from .config import EngineConfig
        return EngineConfig
    raise AttributeError(name)
