from .params import SamplingParams, request_sample_uniform

__all__ = ["SamplingParams", "request_sample_uniform", "Sampler"]


def __getattr__(name):
    if name == "Sampler":
        from .sampler import Sampler
        return Sampler
    raise AttributeError(name)
