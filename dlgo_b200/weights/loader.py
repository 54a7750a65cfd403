"""Weights by tensor name, with one error that says everything that is wrong.

The reference routes tensors by name while reading the file
(models/llm/loader.go:47-71,225-262), silently ignores names it does not know
and never notices a missing tensor at load time.  Here the model says which
tensors it expects (name -> shape); the file is compared against that table up
front, and ONE :class:`WeightError` lists the missing tensors, the unexpected
ones and those of the wrong shape.

Precision: a tensor stored in bfloat16 stays bfloat16 and float16 becomes
bfloat16; a tensor stored in 32-bit floating point stays 32-bit; integer tables
become int32.  Parts then take a copy in their compute precision where it
differs (a float32 run widens bfloat16 matrices, which is exact).
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Tuple

import torch

from .safetensors_io import Checkpoint


class WeightError(ValueError):
    """The weight file does not fit the model."""

    def __init__(self, missing: List[str], unexpected: List[str],
                 wrong_shape: List[Tuple[str, Tuple[int, ...], Tuple[int, ...]]], wrong_type: List[Tuple[str, str]] = ()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_type = list(wrong_type)
        lines = ["weights do not fit the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in self.wrong_shape))
        if self.wrong_type:
            lines.append(f"  wrong type ({len(self.wrong_type)}): " + ", ".join(f"{n} is {t}" for n, t in self.wrong_type))
        super().__init__("\n".join(lines))


def check_against(expected: Mapping[str, Tuple[int, ...]], found: Mapping[str, Tuple[Tuple[int, ...], torch.dtype]]) -> None:
    """Raise one WeightError if ``found`` (name -> (shape, dtype)) is not exactly ``expected``."""
    missing = sorted(n for n in expected if n not in found)
    unexpected = sorted(n for n in found if n not in expected)
    wrong = sorted((n, tuple(found[n][0]), tuple(expected[n])) for n in expected
                   if n in found and tuple(found[n][0]) != tuple(expected[n]))
    bad_type = sorted((n, str(found[n][1])) for n in expected
                      if n in found and not (found[n][1].is_floating_point))
    if missing or unexpected or wrong or bad_type:
        raise WeightError(missing, unexpected, wrong, bad_type)


def stored_precision(t: torch.Tensor) -> torch.Tensor:
    """The loader's precision rule (see module docstring)."""
    if t.dtype in (torch.bfloat16, torch.float32, torch.int32):
        return t
    if t.dtype == torch.float16:
        return t.to(torch.bfloat16)
    if t.dtype == torch.float64:
        return t.to(torch.float32)
    if t.dtype in (torch.int64, torch.int16, torch.int8, torch.uint8, torch.bool):
        return t.to(torch.int32)
    raise ValueError(f"unsupported stored dtype {t.dtype}")


class WeightSource:
    """Tensors of a model folder on the device, read on demand, one device copy per name."""

    def __init__(self, model_dir: str, device: torch.device):
        self.checkpoint = Checkpoint(model_dir)
        self.device = device
        self._cache: Dict[str, torch.Tensor] = {}

    def found(self) -> Dict[str, Tuple[Tuple[int, ...], torch.dtype]]:
        return {n: (self.checkpoint.info(n).shape, self.checkpoint.info(n).dtype) for n in self.checkpoint.names()}

    def get(self, name: str) -> torch.Tensor:
        t = self._cache.get(name)
        if t is None:
            host = self.checkpoint.read(name)
            if self.device.type == "cuda":
                t = stored_precision(host.to(self.device))
            else:
                t = stored_precision(host.clone())
            self._cache[name] = t
        return t

    def release(self) -> None:
        """Drop the by-name references (parts keep what they use)."""
        self._cache.clear()
        self.checkpoint.close()


class DictSource:
    """Tensors given in memory (name -> tensor), with the interface of :class:`WeightSource`."""

    def __init__(self, tensors: Mapping[str, torch.Tensor], device: torch.device):
        self.tensors = dict(tensors)
        self.device = device
        self._cache: Dict[str, torch.Tensor] = {}

    def found(self) -> Dict[str, Tuple[Tuple[int, ...], torch.dtype]]:
        return {n: (tuple(t.shape), t.dtype) for n, t in self.tensors.items()}

    def get(self, name: str) -> torch.Tensor:
        t = self._cache.get(name)
        if t is None:
            t = self._cache[name] = stored_precision(self.tensors[name].to(self.device))
        return t

    def release(self) -> None:
        self._cache.clear()
