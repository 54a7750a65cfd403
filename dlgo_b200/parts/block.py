"""Arrangements of a layer's parts.

``prenorm`` is the reference's standard wiring (models/llm/forward.go:144-169):
``r = x + mixer(norm(x))``, then ``x = r + ffn(norm(r))``.  The residual stream
is one fp32 tensor that mixer and feed-forward add into.
"""
from __future__ import annotations

from typing import Any, Mapping, Optional

import torch

from .base import Block, PositionEncoding
from .registry import BLOCKS


class PreNormBlock(Block):
    def forward(self, residual: torch.Tensor, ctx: Any, cache: Any, state: Optional[torch.Tensor],
                positions: Mapping[str, PositionEncoding]) -> None:
        x = self.mixer_norm.forward(residual)
        self.mixer.forward(x, residual, ctx, cache, state, positions)
        x = self.ffn_norm.forward(residual)
        self.ffn.forward(x, residual, ctx)


BLOCKS.register("prenorm", PreNormBlock)
