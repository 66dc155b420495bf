from .sampler import SamplingParams, choose

__all__ = ["SamplingParams", "choose"]
