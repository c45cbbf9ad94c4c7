from .sampler import Sampler, uniform_draw

__all__ = ["Sampler", "uniform_draw"]
