from .params import SamplingParams, GREEDY, MAX_TOP_K
from .rng import uniform, resolve_seed, splitmix64

__all__ = ["SamplingParams", "GREEDY", "MAX_TOP_K", "uniform", "resolve_seed", "splitmix64"]
