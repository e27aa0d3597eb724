"""Greedy, temperature and nucleus sampling."""

from paged_kv_serving_b200.sampling.sampler import Sampler

__all__ = ["Sampler"]
