from .params import SamplingParams
from .sampler import Sampler, sample_tokens

__all__ = ["SamplingParams", "Sampler", "sample_tokens"]
