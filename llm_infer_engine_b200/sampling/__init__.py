from .sampler import SamplingParams, uniform_for

__all__ = ["SamplingParams", "uniform_for"]
