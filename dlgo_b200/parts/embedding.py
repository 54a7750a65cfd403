"""Token embedding and the output head.

Embedding: ``x = E[token, :]`` with no scaling for this architecture
(models/llm/forward.go:132-135).  Head: ``logits = O . x`` in fp32, with
``O = E`` when the weights are tied (models/llm/forward.go:193-197,
models/llm/loader.go:74-76).
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Optional

import torch

from ..csrc import kernels as K
from .base import ParamSpec, Part
from .linear import STORE_F32, Linear
from .registry import EMBEDDINGS, HEADS


class TokenEmbedding(Part):
    def __init__(self, vocab_size: int, hidden_size: int):
        super().__init__(vocab_size=vocab_size, hidden_size=hidden_size)
        self.vocab_size = int(vocab_size)
        self.hidden_size = int(hidden_size)
        self.table: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.vocab_size, self.hidden_size))}

    def load(self, get: Callable[[str], torch.Tensor], runtime: Any) -> None:
        self.table = runtime.compute_copy(get("weight")).contiguous()

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        return K.embed(token_ids, self.table)


class LinearHead(Part):
    """``tied_to`` names the tensor (absolute name) the head shares, or ``None`` for a weight of its own."""

    def __init__(self, vocab_size: int, hidden_size: int, tied_to: Optional[str] = None):
        super().__init__(vocab_size=vocab_size, hidden_size=hidden_size, tied_to=tied_to)
        self.vocab_size = int(vocab_size)
        self.hidden_size = int(hidden_size)
        self.tied_to = tied_to
        self.proj: Optional[Linear] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {} if self.tied_to else {"weight": ParamSpec((self.vocab_size, self.hidden_size))}

    def load(self, get: Callable[[str], torch.Tensor], runtime: Any) -> None:
        self.proj = Linear(get("weight"), runtime)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.proj(x, STORE_F32)


EMBEDDINGS.register("token_embedding", TokenEmbedding)
HEADS.register("linear_head", LinearHead)
