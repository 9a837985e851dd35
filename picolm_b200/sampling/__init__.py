from .sampler import Sampler, SamplingParams, stream_seed

__all__ = ["Sampler", "SamplingParams", "stream_seed"]
