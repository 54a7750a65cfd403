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


def norm_of(norm: Any, residual: torch.Tensor, ctx: Any) -> torch.Tensor:
    """The norm of the residual stream, adding first whatever the previous part left pending
    (fused into the norm's pass where the norm offers that)."""
    pending = ctx.take_pending() if hasattr(ctx, "take_pending") else None
    if pending is not None:
        if hasattr(norm, "forward_fused"):
            return norm.forward_fused(residual, pending)
        ctx.pending = pending
        ctx.settle(residual)
    return norm.forward(residual)


class PreNormBlock(Block):
    handles_pending = True   # reads the residual only through norm_of

    def __init__(self, mixer: Any, ffn: Any, norms: Mapping[str, Any]):
        super().__init__(mixer, ffn, norms)
        missing = [r for r in ("mixer_norm", "ffn_norm") if r not in self.norms]
        if missing or mixer is None or ffn is None:
            raise ValueError("a pre-norm block needs a mixer, a feed-forward and the norms 'mixer_norm' and 'ffn_norm'"
                             + (f" (missing: {', '.join(missing)})" if missing else ""))
        self.mixer_norm = self.norms["mixer_norm"]
        self.ffn_norm = self.norms["ffn_norm"]

    def forward(self, residual: torch.Tensor, ctx: Any, cache: Any, state: Optional[torch.Tensor],
                positions: Mapping[str, PositionEncoding]) -> None:
        x = norm_of(self.mixer_norm, residual, ctx)
        self.mixer.forward(x, residual, ctx, cache, state, positions)
        x = norm_of(self.ffn_norm, residual, ctx)
        self.ffn.forward(x, residual, ctx)


BLOCKS.register("prenorm", PreNormBlock)
