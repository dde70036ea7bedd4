"""Sampling: parameters and the on-device sampler."""

from .params import SamplingParams

__all__ = ["Sampler", "SamplingParams"]


def __getattr__(name):
    if name == "Sampler":
        from .sampler import Sampler
        return Sampler
    raise AttributeError(name)
