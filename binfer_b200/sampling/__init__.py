"""Sampling: options, per-request random streams, and the device sampler."""
from .params import SamplingParams, uniform
from .sampler import Sampler

__all__ = ["SamplingParams", "uniform", "Sampler"]
