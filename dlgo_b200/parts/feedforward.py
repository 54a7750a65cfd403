"""SwiGLU feed-forward: ``y = Wd . (silu(Wg . x) * (Wu . x))``.

Reference (models/llm/forward.go:293-298): gate and up projections in one
dispatch, ``h = g / (1 + exp(-g)) * u`` (ops/activation.go:8-38), down
projection; the caller adds the result to the residual (:169).  Dense: no
experts, no routing.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Optional

import torch

from ..csrc import kernels as K
from .base import FeedForward, ParamSpec
from .linear import ADD_F32, STORE, Linear
from .registry import FEED_FORWARDS


class SwiGLU(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int):
        super().__init__(hidden_size=hidden_size, intermediate_size=intermediate_size)
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.w_gate_up: Optional[Linear] = None
        self.w_down: Optional[Linear] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {
            "gate_proj.weight": ParamSpec((self.intermediate_size, self.hidden_size)),
            "up_proj.weight": ParamSpec((self.intermediate_size, self.hidden_size)),
            "down_proj.weight": ParamSpec((self.hidden_size, self.intermediate_size)),
        }

    def load(self, get: Callable[[str], torch.Tensor], runtime: Any) -> None:
        gate = runtime.compute_copy(get("gate_proj.weight"))
        up = runtime.compute_copy(get("up_proj.weight"))
        f, d = self.intermediate_size, self.hidden_size
        self.fused = False
        if runtime.dtype == torch.bfloat16 and f % 16 == 0 and d % 8 == 0:
            # blocks of 16 gate rows followed by their 16 up rows: the contraction's epilogue then
            # holds a gate value and its up value side by side and writes silu(g) * u directly
            inter = torch.stack([gate.view(f // 16, 16, d), up.view(f // 16, 16, d)], dim=1).reshape(2 * f, d)
            self.w_gate_up = Linear(inter.contiguous(), runtime, fused_swiglu=True)
            self.fused = True
        else:
            self.w_gate_up = Linear(torch.cat([gate, up], dim=0), runtime)
        self.w_down = Linear(get("down_proj.weight"), runtime)

    def forward(self, x: Any, residual: torch.Tensor, ctx: Any) -> None:
        if self.fused:
            h = self.w_gate_up(x)
        else:
            h = K.swiglu(self.w_gate_up(x, STORE))
        parts = self.w_down.partials(h, for_residual=True) if ctx is not None and hasattr(ctx, "defer") else None
        if parts is not None:
            ctx.defer(residual, parts)      # the next norm adds the slices to the residual
        else:
            self.w_down(h, ADD_F32, residual)


FEED_FORWARDS.register("swiglu", SwiGLU)
