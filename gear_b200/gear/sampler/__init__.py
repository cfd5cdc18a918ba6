from .global_sampler import TopKSampler, UniformSampler, WeightedSampler

__all__ = ["UniformSampler", "WeightedSampler", "TopKSampler"]
