"""Compiling and loading the CUDA kernels.

Each ``.cu`` file of this folder becomes one shared library for sm_100a, built
with ``nvcc`` directly and loaded with ``ctypes``; entry points are plain C
functions that take device pointers, sizes and a stream.  A library is compiled
the first time something needs it (a model asks only for the kernels of its own
parts and precision), into ``_build/`` beside the sources when that folder can
be written, else into a per-user folder under the system's temporary folder.
The file name carries a hash of the sources and flags, so a stale build is
never loaded.  There is no fallback: a kernel that cannot be built or loaded
raises :class:`KernelBuildError`.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from typing import Dict, Iterable, List, Optional

_HERE = os.path.dirname(os.path.abspath(__file__))

# library name -> source files (headers are hashed for all of them)
LIBRARIES: Dict[str, List[str]] = {
    "elementwise": ["elementwise.cu"],
    "gemm_simt": ["gemm_simt.cu"],
    "rope_append": ["rope_append.cu"],
    "attention": ["attention.cu"],
    "sampling": ["sampling.cu"],
    "gemm_tc": ["gemm_tc.cu"],
    "attention_decode": ["attention_decode.cu"],
    "attention_decode_mma": ["attention_decode_mma.cu"],
    "hoststep": ["hoststep.cu"],
    "attention_prefill_tc": ["attention_prefill_tc.cu"],
    "decode_layers": ["decode_layers.cu"],
    "prompt_layers": ["prompt_layers.cu"],
}
_HEADERS = ["common.cuh", "attention_noalloc.h", "attention_combine.cuh", "attention_decode_tiles.cuh", "tcgen05.cuh"]

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class KernelBuildError(RuntimeError):
    pass


def register_library(name: str, sources: List[str]) -> None:
    """Add a library to the table (sources relative to this folder)."""
    LIBRARIES[name] = list(sources)


def _log(msg: str) -> None:
    print(f"[dlgo_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("DLGO_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
                 shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelBuildError("nvcc not found (looked at $DLGO_NVCC, $CUDA_HOME/bin, PATH, /usr/local/cuda/bin)")


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe-{os.getpid()}")
        with open(probe, "w"):
            pass
        os.unlink(probe)
        return True
    except OSError:
        return False


_build_dir_cache: Optional[str] = None


def build_dir() -> str:
    global _build_dir_cache
    if _build_dir_cache:
        return _build_dir_cache
    cands = []
    if os.environ.get("DLGO_BUILD_DIR"):
        cands.append(os.environ["DLGO_BUILD_DIR"])
    cands.append(os.path.join(_HERE, "_build"))
    cands.append(os.path.join(tempfile.gettempdir(), f"dlgo_b200-build-{os.getuid()}"))
    for c in cands:
        if _writable_dir(c):
            _build_dir_cache = c
            return c
    raise KernelBuildError(f"no writable build folder among {cands}")


def _flags() -> List[str]:
    extra = os.environ.get("DLGO_NVCC_FLAGS", "").split()
    return ARCH_FLAGS + BASE_FLAGS + extra


def _digest(name: str) -> str:
    h = hashlib.sha256()
    for rel in LIBRARIES[name] + _HEADERS:
        with open(os.path.join(_HERE, rel), "rb") as f:
            h.update(rel.encode())
            h.update(f.read())
    h.update(" ".join(_flags()).encode())
    return h.hexdigest()[:16]


def library_path(name: str) -> str:
    return os.path.join(build_dir(), f"libdlgo_{name}-{_digest(name)}.so")


def _compile_cmd(name: str, out: str) -> List[str]:
    srcs = [os.path.join(_HERE, s) for s in LIBRARIES[name]]
    return [find_nvcc()] + _flags() + ["-I", _HERE, "-o", out] + srcs + ["-lcudart"]


def ensure_built(names: Iterable[str], verbose: bool = True) -> Dict[str, str]:
    """Compile whichever of ``names`` has no current build; all missing ones in parallel."""
    names = list(dict.fromkeys(names))
    for n in names:
        if n not in LIBRARIES:
            raise KernelBuildError(f"unknown kernel library {n!r}; known: {sorted(LIBRARIES)}")
    paths = {n: library_path(n) for n in names}
    todo = [n for n in names if not os.path.exists(paths[n])]
    if not todo:
        return paths
    procs = []
    t0 = time.time()
    for n in todo:
        tmp = f"{paths[n]}.{os.getpid()}.tmp"
        if verbose:
            _log(f"compiling {n} for sm_100a ({', '.join(LIBRARIES[n])}) ...")
        try:
            p = subprocess.Popen(_compile_cmd(n, tmp), stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        except OSError as e:
            raise KernelBuildError(f"cannot start nvcc: {e}") from None
        procs.append((n, tmp, p))
    last = time.time()
    pending = list(procs)
    errors = []
    while pending:
        for item in list(pending):
            n, tmp, p = item
            if p.poll() is None:
                continue
            out = p.stdout.read() if p.stdout else ""
            pending.remove(item)
            if p.returncode != 0:
                errors.append(f"nvcc failed for {n} (exit {p.returncode}):\n{out}")
                if os.path.exists(tmp):
                    os.unlink(tmp)
            else:
                os.replace(tmp, paths[n])
                if verbose:
                    _log(f"built {n} in {time.time() - t0:.0f} s")
                if out.strip() and os.environ.get("DLGO_NVCC_FLAGS"):
                    _log(out.strip())
        if pending:
            time.sleep(0.2)
            if verbose and time.time() - last > 10:
                last = time.time()
                _log(f"still compiling {', '.join(n for n, _, _ in pending)} ({last - t0:.0f} s)")
    if errors:
        raise KernelBuildError("\n".join(errors))
    return paths


def load_library(name: str, verbose: bool = True) -> ctypes.CDLL:
    """The library's handle; compiled first if need be."""
    with _lock:
        lib = _loaded.get(name)
        if lib is not None:
            return lib
        path = ensure_built([name], verbose=verbose)[name]
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelBuildError(f"cannot load {path}: {e}") from None
        _loaded[name] = lib
        return lib


def load_libraries(names: Iterable[str], verbose: bool = True) -> Dict[str, ctypes.CDLL]:
    names = list(dict.fromkeys(names))
    with _lock:
        missing = [n for n in names if n not in _loaded]
        if missing:
            ensure_built(missing, verbose=verbose)
    return {n: load_library(n, verbose=verbose) for n in names}


def build_all(verbose: bool = True) -> Dict[str, str]:
    """Compile every library (the "does it build" check; needs no GPU)."""
    return ensure_built(sorted(LIBRARIES), verbose=verbose)
