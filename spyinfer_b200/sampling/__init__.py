"""Sampling: per-request options and the device-side sampler."""
from .params import SamplingParams
from .sampler import Sampler

__all__ = ["SamplingParams", "Sampler"]
