"""Sampling: options, host-side state, and the GPU sampler."""

from .config import SamplingConfig
from .host import NgramBlocker, fresh_seed, recent_window, uniform, uniforms

__all__ = ["SamplingConfig", "NgramBlocker", "fresh_seed", "recent_window", "uniform", "uniforms"]
