from .params import SamplingParams
from .rng import SplitMix64
from .sampler import InvalidLogits, Sampler, sample_top_p_host
