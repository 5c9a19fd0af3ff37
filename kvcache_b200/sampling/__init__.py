from .params import SamplingParams
from .sampler import TokenReader

__all__ = ["SamplingParams", "TokenReader"]
