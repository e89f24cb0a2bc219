from .params import GREEDY_TEMPERATURE, SamplingParams
from .rng import uniform

__all__ = ["GREEDY_TEMPERATURE", "SamplingParams", "uniform", "Sampler"]


def __getattr__(name):
    if name == "Sampler":          # needs torch with CUDA only when used
        from .sampler import Sampler
        return Sampler
    raise AttributeError(name)
