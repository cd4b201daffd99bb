"""Sampling: configuration, host chain, device kernels."""
from .sampler import (FunctionSampler, Sampler, SamplerConfig, apply_repeat_penalty, greedy, make_sampler,
                      sample_host, uniform01)

__all__ = ["FunctionSampler", "Sampler", "SamplerConfig", "make_sampler", "apply_repeat_penalty", "greedy", "sample_host", "uniform01"]
