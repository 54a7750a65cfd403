"""Interfaces of the parts a layer is put together from.

A part is built from its constants alone (sizes, eps, theta, ...), declares the
tensors it wants by name, and runs on what the step hands it.  No part knows
which model it is in: the configuration picks parts layer by layer, the model
assembly (engine/model.py) wires them.

Families and what each must offer:

``Norm``              ``forward(residual_f32[T, size]) -> activations[T, size]``
``PositionEncoding``  builds its tables once (``prepare``) and exposes them to
                      the mixers that name it
``Mixer``             ``cache_need()``, ``state_need()``,
                      ``forward(x_normed, residual, ctx, cache, state, positions)``
                      which ADDS its result into ``residual`` (fp32, in place)
``FeedForward``       ``forward(x_normed, residual, ctx)``, same contract
``Block``             the arrangement of the above in one layer

The residual stream is fp32 in every precision; activations between kernels are
in the run's dtype (bfloat16 or float32).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping, Optional, Tuple

import torch


@dataclass(frozen=True)
class ParamSpec:
    """One tensor a part wants from the weight file.

    ``init`` says how the random-weights mode fills it: ``"normal"`` is
    N(0, std), ``"one_plus_normal"`` is 1 + N(0, std) (norm weights).
    """

    shape: Tuple[int, ...]
    init: str = "normal"


@dataclass(frozen=True)
class CacheNeed:
    """What a mixer keeps per position of a sequence.

    Entries of the run order whose needs are equal and that name the same
    ``group`` share one allocation.  ``window`` (positions) is ``None`` for
    "all keys"; a windowed group gives pages back once every position in them
    lies outside the window of all queries still to come.
    """

    group: str
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """Fixed-size state a mixer keeps per sequence: zeroed when a slot is taken.

    In the spirit of the reference's ``SSMLayerState`` (memory/ssmstate.go:4-41),
    allocated only for layers that ask for it (models/llm/forward.go:89-109).
    """

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Part:
    """Base of all parts: constants in, named tensors wanted, nothing else."""

    def __init__(self, **params: Any):
        self.params = dict(params)

    def param_specs(self) -> Dict[str, ParamSpec]:
        """Tensors wanted, by name relative to the part's prefix."""
        return {}

    def load(self, get: Callable[[str], torch.Tensor], runtime: "Any") -> None:
        """Take the tensors (``get(relative_name)`` returns them on the device in
        their stored precision) and prepare them for ``runtime.dtype``."""

    def prepare(self, runtime: "Any") -> None:
        """Build tables that depend on constants only."""


class Norm(Part):
    def forward(self, residual: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    pass


class Mixer(Part):
    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def state_need(self) -> Optional[StateNeed]:
        return None

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: "Any", cache: "Any",
                state: Optional[torch.Tensor], positions: Mapping[str, PositionEncoding]) -> None:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: "Any") -> None:
        raise NotImplementedError


class Block:
    """Arrangement of one layer's parts.

    ``norms`` maps the role names of the layer's description to the norms built for them, as many as
    the arrangement reads; ``mixer`` or ``ffn`` is ``None`` where the layer has none.  A subclass's
    ``forward`` decides who reads the residual stream when.
    """

    def __init__(self, mixer: Optional[Mixer], ffn: Optional[FeedForward], norms: Mapping[str, Norm]):
        self.mixer = mixer
        self.ffn = ffn
        self.norms: Dict[str, Norm] = dict(norms)

    def parts(self) -> Dict[str, Part]:
        """Every part of the layer by role (norm roles, ``mixer``, ``ffn``): what holds its tensors."""
        out: Dict[str, Part] = dict(self.norms)
        if self.mixer is not None:
            out["mixer"] = self.mixer
        if self.ffn is not None:
            out["ffn"] = self.ffn
        return out

    def forward(self, residual: torch.Tensor, ctx: "Any", cache: "Any", state: Optional[torch.Tensor],
                positions: Mapping[str, PositionEncoding]) -> None:
        raise NotImplementedError
