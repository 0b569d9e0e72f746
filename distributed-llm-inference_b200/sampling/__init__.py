from .params import SamplingParams
from .sampler import PendingTokens, Sampler, SamplerState

__all__ = ["PendingTokens", "Sampler", "SamplerState", "SamplingParams"]
