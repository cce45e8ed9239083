from .sampler import Sampler, SamplingParams, SamplingState

__all__ = ["Sampler", "SamplingParams", "SamplingState"]
