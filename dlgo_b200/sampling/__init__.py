"""Choosing the next token: sampler configuration and the device sampler."""
from .sampler import DeviceSampler, RECENT_WINDOW, SamplerConfig

__all__ = ["DeviceSampler", "RECENT_WINDOW", "SamplerConfig"]
