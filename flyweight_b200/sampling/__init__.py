from .config import GREEDY, SamplingConfig
from .rng import XorShift64Star

__all__ = ["GREEDY", "SamplingConfig", "XorShift64Star"]
