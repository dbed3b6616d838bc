from .params import SamplingParams
from .sampler import Sampler, recent_tokens, stream_of

__all__ = ["SamplingParams", "Sampler", "recent_tokens", "stream_of"]
