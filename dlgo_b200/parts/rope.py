"""Rotary position encoding: cos/sin tables built once from constants.

Reference: ``theta_i = base^(-2i/rotary_dim)``, ``angle = pos * theta_i`` in
float64, cos and sin cast to float32, one row per position
(models/llm/workers.go:147-171); only the first ``rotary_dim`` dims of a head
are rotated (workers.go:151-159).  Pairing: ``split_half`` pairs (i, i+rot/2),
``interleaved`` pairs (2i, 2i+1) (ops/rope.go:21-31); which one is right is a
property of the weight layout, so it is a parameter.

The llama3 scaling of the frequencies is not in the reference (it has no rope
scaling at all); it follows the published Llama 3.1 rule: with wavelength
``lam = 2*pi/f``, frequencies with ``lam < orig/high`` are kept, those with
``lam > orig/low`` are divided by ``factor``, and those between are blended by
``s = (orig/lam - low) / (high - low)``: ``f <- (1-s) * f/factor + s * f``.
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional

import torch

from .base import PositionEncoding
from .registry import POSITION_ENCODINGS


def rotary_frequencies(rotary_dim: int, theta: float, scaling: Optional[Dict[str, Any]]) -> List[float]:
    half = rotary_dim // 2
    freqs = [1.0 / math.pow(theta, (2 * i) / rotary_dim) for i in range(half)]
    if not scaling:
        return freqs
    kind = scaling.get("rope_type", "llama3")
    if kind != "llama3":
        raise ValueError(f"rotary scaling {kind!r} is not supported")
    factor = float(scaling["factor"])
    low = float(scaling["low_freq_factor"])
    high = float(scaling["high_freq_factor"])
    orig = float(scaling["original_max_position_embeddings"])
    out = []
    for f in freqs:
        lam = 2.0 * math.pi / f
        if lam < orig / high:
            out.append(f)
        elif lam > orig / low:
            out.append(f / factor)
        else:
            s = (orig / lam - low) / (high - low)
            out.append((1.0 - s) * f / factor + s * f)
    return out


class RotaryEmbedding(PositionEncoding):
    def __init__(self, head_dim: int, rotary_dim: int, theta: float, max_positions: int,
                 pairing: str = "split_half", scaling: Optional[Dict[str, Any]] = None):
        super().__init__(head_dim=head_dim, rotary_dim=rotary_dim, theta=theta, max_positions=max_positions,
                         pairing=pairing, scaling=scaling)
        if rotary_dim % 2 or not 0 < rotary_dim <= head_dim:
            raise ValueError(f"rotary_dim must be even and in (0, head_dim], got {rotary_dim} for head_dim {head_dim}")
        if pairing not in ("split_half", "interleaved"):
            raise ValueError(f"pairing must be 'split_half' or 'interleaved', got {pairing!r}")
        self.head_dim = int(head_dim)
        self.rotary_dim = int(rotary_dim)
        self.theta = float(theta)
        self.max_positions = int(max_positions)
        self.interleaved = pairing == "interleaved"
        self.scaling = dict(scaling) if scaling else None
        self.cos: Optional[torch.Tensor] = None
        self.sin: Optional[torch.Tensor] = None

    def tables(self) -> tuple[torch.Tensor, torch.Tensor]:
        """(cos, sin), each ``[max_positions, rotary_dim/2]`` float32 on the CPU."""
        f = torch.tensor(rotary_frequencies(self.rotary_dim, self.theta, self.scaling), dtype=torch.float64)
        pos = torch.arange(self.max_positions, dtype=torch.float64)
        ang = pos[:, None] * f[None, :]
        return torch.cos(ang).to(torch.float32), torch.sin(ang).to(torch.float32)

    def prepare(self, runtime: Any) -> None:
        c, s = self.tables()
        self.cos = c.contiguous().to(runtime.device)
        self.sin = s.contiguous().to(runtime.device)


POSITION_ENCODINGS.register("rotary", RotaryEmbedding)
