"""Reading and writing the safetensors container.

The format: an 8-byte little-endian header length, a JSON header
``{name: {"dtype", "shape", "data_offsets": [begin, end]}}`` (plus an optional
``__metadata__`` entry), then the raw little-endian tensor bytes.  This takes
the place of the reference's GGUF parser (format/gguf/gguf.go:132) and of
``readTensorData`` (models/llm/loader.go:127-140): a tensor is found by name and
read at its offset.  Files are memory-mapped; a tensor's bytes are touched only
when it is asked for.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Mapping, Tuple

import torch

_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    """A file that is not a well-formed safetensors container."""


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    begin: int
    end: int
    file: str


class SafetensorsFile:
    """One memory-mapped safetensors file."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"{path}: cannot open ({e.strerror})") from None
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: truncated (no header length)")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen > size - 8:
            raise SafetensorsError(f"{path}: truncated (header of {hlen} bytes does not fit in {size} bytes)")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        self.metadata = header.pop("__metadata__", {}) or {}
        self._data_start = 8 + hlen
        data_size = size - self._data_start
        self.tensors: Dict[str, TensorInfo] = {}
        for name, ent in header.items():
            try:
                dt = ent["dtype"]
                shape = tuple(int(s) for s in ent["shape"])
                begin, end = (int(x) for x in ent["data_offsets"])
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed header entry for {name!r}") from None
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dt!r}")
            n = 1
            for s in shape:
                n *= s
            if end - begin != n * _DTYPES[dt][1] or begin < 0:
                raise SafetensorsError(f"{path}: tensor {name!r}: {end - begin} bytes for shape {list(shape)} {dt}")
            if end > data_size:
                raise SafetensorsError(f"{path}: truncated (tensor {name!r} ends at byte {end} of {data_size})")
            self.tensors[name] = TensorInfo(name, _DTYPES[dt][0], shape, begin, end, path)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def read(self, name: str) -> torch.Tensor:
        """The tensor as a CPU tensor that views the mapped file (read-only: copy before writing)."""
        info = self.tensors[name]
        n = 1
        for s in info.shape:
            n *= s
        if n == 0:
            return torch.empty(info.shape, dtype=info.dtype)
        buf = memoryview(self._mm)[self._data_start + info.begin:self._data_start + info.end]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # torch warns that the buffer is not writable
            t = torch.frombuffer(buf, dtype=info.dtype, count=n)
        return t.reshape(info.shape)

    def close(self) -> None:
        # Tensors handed out may still view the mapping; let the garbage collector
        # unmap once they are gone.
        self._mm = None
        self._f.close()


class Checkpoint:
    """All tensors of a model folder: ``model.safetensors`` or the shards its index names."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        single = os.path.join(model_dir, "model.safetensors")
        index = os.path.join(model_dir, "model.safetensors.index.json")
        paths: List[str]
        if os.path.exists(single):
            paths = [single]
        elif os.path.exists(index):
            with open(index, "r", encoding="utf-8") as f:
                try:
                    wm = json.load(f)["weight_map"]
                except (json.JSONDecodeError, KeyError, TypeError):
                    raise SafetensorsError(f"{index}: no weight_map") from None
            paths = [os.path.join(model_dir, p) for p in sorted(set(wm.values()))]
        else:
            raise SafetensorsError(f"{model_dir}: neither model.safetensors nor model.safetensors.index.json found")
        self.files = [SafetensorsFile(p) for p in paths]
        self.tensors: Dict[str, Tuple[SafetensorsFile, TensorInfo]] = {}
        for sf in self.files:
            for name, info in sf.tensors.items():
                if name in self.tensors:
                    raise SafetensorsError(f"tensor {name!r} appears in {self.tensors[name][1].file} and {sf.path}")
                self.tensors[name] = (sf, info)

    def names(self) -> List[str]:
        return sorted(self.tensors)

    def info(self, name: str) -> TensorInfo:
        return self.tensors[name][1]

    def read(self, name: str) -> torch.Tensor:
        sf, _ = self.tensors[name]
        return sf.read(name)

    def close(self) -> None:
        for sf in self.files:
            sf.close()


def write_safetensors(path: str, tensors: Iterable[Tuple[str, Tuple[int, ...], torch.dtype]],
                      produce, metadata: Mapping[str, str] | None = None) -> None:
    """Write a file tensor by tensor.

    ``tensors`` lists (name, shape, dtype) in file order; ``produce(name)`` returns
    that tensor (any device) when its turn comes, so a model larger than host
    memory to spare is never held twice.
    """
    entries = list(tensors)
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    off = 0
    for name, shape, dtype in entries:
        if dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {dtype} for tensor {name!r}")
        n = 1
        for s in shape:
            n *= s
        nbytes = n * _DTYPES[_NAMES[dtype]][1]
        header[name] = {"dtype": _NAMES[dtype], "shape": list(shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name, shape, dtype in entries:
            t = produce(name)
            if tuple(t.shape) != tuple(shape) or t.dtype != dtype:
                raise SafetensorsError(
                    f"tensor {name!r}: produced {list(t.shape)} {t.dtype}, declared {list(shape)} {dtype}")
            t = t.detach().contiguous().cpu()
            if t.numel():
                f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes())
    os.replace(tmp, path)


def save_tensors(path: str, tensors: Mapping[str, torch.Tensor], metadata: Mapping[str, str] | None = None) -> None:
    """Write a dict of tensors (names in sorted order)."""
    names = sorted(tensors)
    write_safetensors(path, [(n, tuple(tensors[n].shape), tensors[n].dtype) for n in names],
                      lambda n: tensors[n], metadata)
