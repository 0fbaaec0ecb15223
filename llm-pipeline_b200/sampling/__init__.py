"""Greedy and temperature sampling with top-k, top-p, min-p, typical-p and repetition penalty."""

from .sampler import Sampler, SamplingConfig, pack_rows, uniform_of

__all__ = ["Sampler", "SamplingConfig", "pack_rows", "uniform_of"]
