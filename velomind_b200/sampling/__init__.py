from .sampler import DeviceSampler, SamplingParams

__all__ = ["DeviceSampler", "SamplingParams"]
