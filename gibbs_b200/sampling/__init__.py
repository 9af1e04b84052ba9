from .params import (DEFAULT_MAX_NEW_TOKENS, DEFAULT_TEMPERATURE, DEFAULT_TOP_K, DEFAULT_TOP_P, GREEDY_BELOW,
                     MAX_TOP_K, SamplingParams, TokenLogprobInfo)
from .sampler import Sampler, uniform24

__all__ = ["SamplingParams", "TokenLogprobInfo", "Sampler", "uniform24", "DEFAULT_MAX_NEW_TOKENS", "DEFAULT_TEMPERATURE",
           "DEFAULT_TOP_K", "DEFAULT_TOP_P", "GREEDY_BELOW", "MAX_TOP_K"]
