"""Greedy, temperature and filtered sampling."""
from .sampler import (DeviceSampler, RECENT_WINDOW, SamplerConfig, apply_min_p, apply_repetition_penalty, apply_top_k,
                      apply_top_p)

__all__ = ["DeviceSampler", "RECENT_WINDOW", "SamplerConfig", "apply_min_p", "apply_repetition_penalty",
           "apply_top_k", "apply_top_p"]
