"""Architecture description as data.

A configuration class (one per architecture) turns its ``config.json`` keys
into an :class:`ArchitectureSpec`.  Everything below the configuration - the
weight loader, the cache, the model assembly and the step function - reads only
this description; none of them knows which architecture it serves.

The reference resolves a ``LayerSpec{Norm, Core, Residual, FFN, ...}`` for every
layer at load time (models/llm/model.go:48-56, models/llm/loader.go:88-125) and
switches on it in the forward pass (models/llm/forward.go:142-182).  Here the
same idea is carried further: each part of a layer is named by a registry key
plus its constants, layer by layer, and the order in which layers run is a list
of its own.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Sequence


@dataclass(frozen=True)
class PartSpec:
    """One part of a model: a registry key and the constants it is built with."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def with_params(self, **more: Any) -> "PartSpec":
        merged = dict(self.params)
        merged.update(more)
        return PartSpec(self.kind, merged)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement ("block") of a mixer, a feed-forward and norms.

    ``norms`` maps a role name to a norm, as many as the block reads: the
    pre-norm block reads ``mixer_norm`` and ``ffn_norm``; a block with norms
    after its parts as well (the reference's ``PostAttnNorm`` / ``PostFFNNorm``,
    models/llm/forward.go:158-182) names four.  ``mixer`` or ``ffn`` may be
    ``None`` for a block that has no such part.  ``prefix`` is the layer's
    tensor-name prefix in the weight file; ``names`` maps each role (``mixer``,
    ``ffn`` and every norm role) to the sub-prefix its tensors carry below
    ``prefix``.
    """

    prefix: str
    block: str
    mixer: Optional[PartSpec]
    ffn: Optional[PartSpec]
    norms: Mapping[str, PartSpec]
    names: Mapping[str, str]

    def roles(self) -> Sequence[str]:
        """Every role of the layer that has a part, norms first in their own order."""
        out = list(self.norms)
        if self.mixer is not None:
            out.append("mixer")
        if self.ffn is not None:
            out.append("ffn")
        return out


@dataclass(frozen=True)
class RunEntry:
    """One entry of the run order.

    ``layer`` indexes :attr:`ArchitectureSpec.layers`; the same layer may appear
    in several entries (its weights are then shared, its cache is not).
    ``cache_of`` names an EARLIER entry of the order whose cache this entry
    reads instead of keeping one of its own; ``None`` means its own.
    """

    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ArchitectureSpec:
    name: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    embedding_prefix: str
    layers: Sequence[LayerSpec]
    order: Sequence[RunEntry]
    final_norm: PartSpec
    final_norm_prefix: str
    head: PartSpec
    head_prefix: str
    position_encodings: Mapping[str, PartSpec]
    bos_token_id: Optional[int]
    stop_token_ids: Sequence[int]

    def validate(self) -> None:
        n = len(self.layers)
        if n == 0:
            raise ValueError("architecture has no layers")
        if not self.order:
            raise ValueError("architecture has an empty run order")
        for j, ls in enumerate(self.layers):
            missing = [r for r in ls.roles() if r not in ls.names]
            if missing:
                raise ValueError(f"layer {j}: no tensor-name prefix for the role(s) {', '.join(missing)}")
            if set(ls.norms) & {"mixer", "ffn"}:
                raise ValueError(f"layer {j}: a norm cannot take the role name 'mixer' or 'ffn'")
        for i, e in enumerate(self.order):
            if not 0 <= e.layer < n:
                raise ValueError(f"run entry {i} names layer {e.layer}, but there are {n} layers")
            if e.cache_of is not None:
                if not 0 <= e.cache_of < i:
                    raise ValueError(
                        f"run entry {i} reads the cache of entry {e.cache_of}, which does not come before it")
                if self.order[e.cache_of].cache_of is not None:
                    raise ValueError(
                        f"run entry {i} reads the cache of entry {e.cache_of}, which itself borrows a cache")
