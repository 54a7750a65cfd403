"""RMSNorm: ``out = x * (1 / sqrt(mean(x^2) + eps)) * w`` (ops/norm.go:10-32),
statistics in fp32 on the fp32 residual stream, output in the run's precision."""
from __future__ import annotations

from typing import Any, Callable, Dict, Optional

import torch

from ..csrc import kernels as K
from .base import Norm, ParamSpec
from .registry import NORMS


class RMSNorm(Norm):
    def __init__(self, size: int, eps: float):
        super().__init__(size=size, eps=eps)
        self.size = int(size)
        self.eps = float(eps)
        self.weight: Optional[torch.Tensor] = None
        self.out_dtype: Optional[torch.dtype] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.size,), "one_plus_normal")}

    def load(self, get: Callable[[str], torch.Tensor], runtime: Any) -> None:
        self.weight = runtime.compute_copy(get("weight"), torch.float32).contiguous()
        self.out_dtype = runtime.dtype

    def forward(self, residual: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        return K.rmsnorm(residual, self.weight, self.eps, self.out_dtype, rows)

    def forward_fused(self, residual: torch.Tensor, parts: torch.Tensor,
                      rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``residual += parts.sum(0)`` and the norm of the new rows, in one pass."""
        return K.add_rmsnorm(residual, parts, self.weight, self.eps, self.out_dtype, rows)


NORMS.register("rmsnorm", RMSNorm)
