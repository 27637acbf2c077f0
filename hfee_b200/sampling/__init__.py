from .options import SamplingOptions
from .sampler import BatchSampler, apply_repeat_penalty, fresh_seed, sample_host, uniform

__all__ = ["SamplingOptions", "BatchSampler", "apply_repeat_penalty", "fresh_seed", "sample_host", "uniform"]
