from .params import SamplingParams
from .sampler import PendingTokens, Sampler

__all__ = ["PendingTokens", "Sampler", "SamplingParams"]
