from .params import DEFAULT_SEED, MAX_TOP_K, SamplingParams
from .sampler import BatchSampler

__all__ = ["DEFAULT_SEED", "MAX_TOP_K", "SamplingParams", "BatchSampler"]
