from .config import SamplingConfig
from .sampler import Sampler, fresh_seed

__all__ = ["Sampler", "SamplingConfig", "fresh_seed"]
