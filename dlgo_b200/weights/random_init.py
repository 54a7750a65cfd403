"""Random-weights mode: a model folder (config.json, model.safetensors) from a configuration and a seed.

The reference has no such mode (its tests need real model files,
models/llm/llm_test.go:10-23).  Every matrix and the embedding are N(0, std),
norm weights are 1 + N(0, std), std 0.02 by default; the tensors are those the
model built from the configuration expects, in sorted name order, each drawn
from one generator seeded with ``seed`` in that order, so the folder is a pure
function of (configuration, seed, std, dtype, device kind).
"""
from __future__ import annotations

import json
import os
from typing import Any, Optional

import torch

from .safetensors_io import write_safetensors


def write_random_model(config: Any, seed: int, out_dir: str, std: float = 0.02,
                       dtype: torch.dtype = torch.bfloat16, device: Optional[str] = None) -> str:
    """Write ``out_dir/config.json`` and ``out_dir/model.safetensors``; returns ``out_dir``.

    ``device`` is where the numbers are drawn ("cpu" by default; "cuda" is much
    faster for large models but draws a different stream).
    """
    from ..engine.model import CausalLM

    if dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("random weights are stored as bfloat16 or float32")
    model = CausalLM(config.architecture_spec())
    expected = model.expected_tensors()
    names = sorted(expected)
    dev = torch.device(device or "cpu")
    gen = torch.Generator(device=dev)
    gen.manual_seed(int(seed))

    def produce(name: str) -> torch.Tensor:
        spec = expected[name]
        t = torch.randn(spec.shape, generator=gen, device=dev, dtype=torch.float32) * std
        if spec.init == "one_plus_normal":
            t = t + 1.0
        elif spec.init != "normal":
            raise ValueError(f"tensor {name!r}: unknown init {spec.init!r}")
        return t.to(dtype)

    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config.to_dict(), f, indent=2)
    write_safetensors(os.path.join(out_dir, "model.safetensors"),
                      [(n, tuple(expected[n].shape), dtype) for n in names], produce,
                      metadata={"format": "pt", "seed": str(seed), "std": repr(std)})
    return out_dir
