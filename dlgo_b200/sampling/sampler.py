"""Choosing the next token.

The reference's pipeline (ops/sampling.go:32-48): greedy if the temperature is
<= 0, else repetition penalty over the recent tokens (:53-69), temperature
(:72-80), top-k (:83-95), top-p (:99-138), min-p (:143-165), softmax and an
inverse-CDF draw (:167-181).  Defaults 0.7 / 40 / 0.9 / 0 / 1.1 (:19-27).

Greedy, the temperature draw and all filters are CUDA kernels of this package
(csrc/sampling.cu); only token ids leave the device.  Filters set logits to
-inf, which the draw treats as probability zero.

The uniform number of a draw is a counter-based function of (seed, request
index, index of the draw within the request), so what a request samples does
not depend on which other requests share its batch.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from ..csrc import kernels as K


@dataclass(frozen=True)
class SamplerConfig:
    temperature: float = 0.7
    top_k: int = 40
    top_p: float = 0.9
    min_p: float = 0.0
    repetition_penalty: float = 1.1

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0

    @property
    def filtered(self) -> bool:
        return self.top_k > 0 or self.top_p < 1.0 or self.min_p > 0 or self.repetition_penalty > 1.0

    @staticmethod
    def greedy_config() -> "SamplerConfig":
        return SamplerConfig(temperature=0.0, top_k=0, top_p=1.0, min_p=0.0, repetition_penalty=1.0)

    @staticmethod
    def plain_temperature(t: float) -> "SamplerConfig":
        return SamplerConfig(temperature=t, top_k=0, top_p=1.0, min_p=0.0, repetition_penalty=1.0)


RECENT_WINDOW = 64  # tokens the repetition penalty looks back over (models/llm/generate.go:143)


def temperature_rows(cfg: SamplerConfig, rows: int, device: torch.device) -> torch.Tensor:
    """The per-row temperature the draw divides by: the filters already applied it, if there are any."""
    return torch.full((rows,), 1.0 if cfg.filtered else float(cfg.temperature), dtype=torch.float32, device=device)


def draw_on_device(logits: torch.Tensor, cfg: SamplerConfig, requests: torch.Tensor, draws: torch.Tensor,
                   recent: Optional[torch.Tensor], seed: int, seed_dev: Optional[torch.Tensor] = None,
                   out: Optional[torch.Tensor] = None, temperature: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Filters and the draw for a sampled (not greedy) configuration, everything already on the device:
    ``requests`` and ``draws`` int32 [rows], ``recent`` int32 [rows, <= 64] with -1 for none (or ``None``).
    ``seed_dev``: the seed is read from device memory (a captured step); ``temperature``: the constant of
    :func:`temperature_rows`, made once by a caller that runs this many times."""
    rows = logits.shape[0]
    if temperature is None:
        temperature = temperature_rows(cfg, rows, logits.device)
    if cfg.filtered:
        # every filter in one kernel of ours; top-k off (0, or at least the vocabulary) is a path of its own there
        top_k = cfg.top_k if 0 < cfg.top_k < logits.shape[1] else 0
        if top_k > K.FILTER_MAX_K:
            raise ValueError(f"top_k up to {K.FILTER_MAX_K} (or 0 for none), got {cfg.top_k}")
        rec = recent if cfg.repetition_penalty > 1.0 else None
        if K.filter_draw_chunks(logits.shape[1], top_k) > 0:
            # a small top-k: only what it can keep is looked at
            return K.filter_draw(logits, cfg.temperature, top_k, cfg.top_p, cfg.min_p, cfg.repetition_penalty, rec,
                                 requests, draws, seed, out, seed_dev)
        work = K.filter_logits(logits, cfg.temperature, top_k, cfg.top_p, cfg.min_p, cfg.repetition_penalty, rec)
        return K.sample(work, temperature, requests, draws, seed, out, seed_dev)
    return K.sample(logits, temperature, requests, draws, seed, out, seed_dev)


class DeviceSampler:
    """Samples one token per row of a logits tensor, on the device."""

    def __init__(self, seed: int = 0):
        self.seed = int(seed)

    def sample(self, logits: torch.Tensor, cfg: SamplerConfig, requests: Sequence[int], draws: Sequence[int],
               recent: Optional[Sequence[Sequence[int]]] = None) -> torch.Tensor:
        """``logits`` [rows, vocab] fp32 on the device -> int32 [rows] on the device."""
        if cfg.greedy:
            return K.argmax(logits)
        dev = logits.device
        meta = torch.tensor([list(requests), list(draws)], dtype=torch.int32).to(dev, non_blocking=True)
        rec = None
        if cfg.filtered and recent is not None and cfg.repetition_penalty > 1.0:
            width = min(RECENT_WINDOW, K.FILTER_MAX_RECENT)
            rec = torch.tensor([(list(r)[-width:] + [-1] * width)[:width] for r in recent],
                               dtype=torch.int32).to(dev, non_blocking=True)
        return draw_on_device(logits, cfg, meta[0], meta[1], rec, self.seed)
