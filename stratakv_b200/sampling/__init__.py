from .sampler import Sampler, SamplingParams

__all__ = ["Sampler", "SamplingParams"]
