"""Sampling: configuration, host chain, device kernels."""
from .sampler import Sampler, SamplerConfig, apply_repeat_penalty, greedy, sample_host, uniform01

__all__ = ["Sampler", "SamplerConfig", "apply_repeat_penalty", "greedy", "sample_host", "uniform01"]
