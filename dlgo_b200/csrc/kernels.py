"""Python face of the CUDA entry points: tensors in, checked, launched on the
current stream.  Nothing here computes; a missing or failing library raises."""
from __future__ import annotations

import ctypes
from typing import Sequence, List, Optional

import torch

from . import build

F32, BF16 = 0, 1
_STATUS = {
    -1: "a size this kernel does not take",
    -2: "a pointer or stride that breaks an alignment rule",
    -3: "an element type this kernel does not take",
    -4: "a CUDA driver entry point could not be found",
    -5: "the kernel gave up a bounded wait on the device",
}


class KernelError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, not {dt}")


LAUNCHES = 0  # kernels of this package launched (or captured into a graph) so far

# Per-kernel timing a user can switch on (the reference's DLGO_PROFILE, examples/benchmark/main.go:24-28): while
# on, a CUDA event follows every launch of this package; the time between two consecutive events is the time of
# the later launch (kernels of one stream run in order).  Meant for runs without CUDA graphs.
_profile_events: Optional[list] = None


def profile_start() -> None:
    """Begin timing every launch of this package on the current stream."""
    global _profile_events
    first = torch.cuda.Event(enable_timing=True)
    first.record()
    _profile_events = [("", first)]


def profile_stop() -> List[tuple]:
    """End the timing; returns [(entry point, launches, total ms)] sorted by time, most first."""
    global _profile_events
    events, _profile_events = _profile_events or [], None
    if len(events) < 2:
        return []
    torch.cuda.synchronize()
    total: dict = {}
    for (_, before), (name, after) in zip(events, events[1:]):
        n, ms = total.get(name, (0, 0.0))
        total[name] = (n + 1, ms + before.elapsed_time(after))
    return sorted(((k, n, ms) for k, (n, ms) in total.items()), key=lambda r: -r[2])


def _check(status: int, what: str, launches: int = 1) -> None:
    global LAUNCHES
    if status == 0:
        LAUNCHES += launches
        if _profile_events is not None and launches > 0 and not torch.cuda.is_current_stream_capturing():
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            _profile_events.append((what, ev))
        return
    if status < 0:
        raise KernelError(f"{what}: refused ({_STATUS.get(status, status)})")
    raise KernelError(f"{what}: CUDA error {status} at launch")


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream() -> ctypes.c_void_p:
    # the raw handle of the current stream of the current device (a C call; current_stream() builds objects)
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice()))


def _need(t: torch.Tensor, dt: Optional[torch.dtype], name: str) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must live on the GPU (there is no CPU path)")
    if dt is not None and t.dtype != dt:
        raise KernelError(f"{name} must be {dt}, is {t.dtype}")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


def _lib(name: str) -> ctypes.CDLL:
    return build.load_library(name)


_i, _f, _p, _ll = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_longlong


# ------------------------------------------------------------------ elementwise
def embed(tokens: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t, :] = table[tokens[t], :] as fp32."""
    _need(tokens, torch.int32, "tokens")
    _need(table, None, "table")
    T, (V, d) = tokens.numel(), table.shape
    if out is None:
        out = torch.empty((T, d), dtype=torch.float32, device=table.device)
    _need(out, torch.float32, "out")
    st = _lib("elementwise").dlgo_embed(_ptr(tokens), _ptr(table), _i(dtype_code(table.dtype)), _ptr(out), _i(T), _i(d),
                                        _i(V), _stream())
    _check(st, "embed")
    return out


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, out_dtype: torch.dtype,
            rows: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Row-wise RMSNorm of fp32 ``x``; with ``rows`` only those rows, in that order."""
    _need(x, torch.float32, "x")
    _need(w, torch.float32, "w")
    d = x.shape[-1]
    if w.numel() != d:
        raise KernelError(f"rmsnorm: weight has {w.numel()} elements, rows have {d}")
    R = x.shape[0] if rows is None else rows.numel()
    if rows is not None:
        _need(rows, torch.int32, "rows")
    if out is None:
        out = torch.empty((R, d), dtype=out_dtype, device=x.device)
    _need(out, out_dtype, "out")
    st = _lib("elementwise").dlgo_rmsnorm(_ptr(x), _ptr(w), _ptr(out), _i(dtype_code(out_dtype)), _ptr(rows), _i(R),
                                          _i(d), _f(eps), _stream())
    _check(st, "rmsnorm")
    return out


def add_rmsnorm(x: torch.Tensor, parts: torch.Tensor, w: Optional[torch.Tensor], eps: float,
                out_dtype: Optional[torch.dtype], rows: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """``x += parts.sum(0)`` (slices in order, in place), then RMSNorm of the new rows; with ``w`` None
    only the sum.  ``parts`` is [S, T, d] fp32."""
    _need(x, torch.float32, "x")
    if parts.dtype != torch.float32 or parts.dim() != 3 or parts.stride(2) != 1 or parts.stride(1) != x.shape[1]:
        raise KernelError("add_rmsnorm: parts must be [S, T, d] float32 with contiguous rows")
    d = x.shape[-1]
    R = x.shape[0] if rows is None else rows.numel()
    out = None
    if w is not None:
        _need(w, torch.float32, "w")
        out = torch.empty((R, d), dtype=out_dtype, device=x.device)
    if rows is not None:
        _need(rows, torch.int32, "rows")
    st = _lib("elementwise").dlgo_add_rmsnorm(
        _ptr(x), _ptr(parts), _i(parts.shape[0]), _ll(parts.stride(0)), _ptr(w), _ptr(out),
        _i(dtype_code(out_dtype) if w is not None else F32), _ptr(rows), _i(R), _i(d), _f(eps), _stream())
    _check(st, "add_rmsnorm")
    return out


def swiglu(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """[T, 2F] (gate | up) -> [T, F]."""
    _need(gate_up, None, "gate_up")
    T, F2 = gate_up.shape
    F = F2 // 2
    if out is None:
        out = torch.empty((T, F), dtype=gate_up.dtype, device=gate_up.device)
    _need(out, gate_up.dtype, "out")
    st = _lib("elementwise").dlgo_swiglu(_ptr(gate_up), _ptr(out), _i(dtype_code(gate_up.dtype)), _i(T), _i(F),
                                         _stream())
    _check(st, "swiglu")
    return out


# ------------------------------------------------------------------------ GEMM
EPI_STORE, EPI_STORE_F32, EPI_ADD_F32 = 0, 1, 2


def gemm_simt(x: torch.Tensor, w: torch.Tensor, epilogue: int = EPI_STORE,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x[M, K] . w[N, K]^T on the fp32 pipes; epilogue stores (x's type or fp32) or adds into fp32 ``out``."""
    _need(w, x.dtype, "w")
    if x.dim() != 2 or x.stride(1) != 1:
        raise KernelError("gemm: x must be 2-D with unit inner stride")
    M, K = x.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelError(f"gemm: x has K={K}, w has K={K2}")
    if out is None:
        if epilogue == EPI_ADD_F32:
            raise KernelError("gemm: the add epilogue needs the tensor to add into")
        out = torch.empty((M, N), dtype=x.dtype if epilogue == EPI_STORE else torch.float32, device=x.device)
    if out.dim() != 2 or out.stride(1) != 1 or out.shape != (M, N):
        raise KernelError(f"gemm: out must be [{M}, {N}] with unit inner stride")
    want = x.dtype if epilogue == EPI_STORE else torch.float32
    if out.dtype != want:
        raise KernelError(f"gemm: out must be {want}")
    st = _lib("gemm_simt").dlgo_gemm_simt(_ptr(x), _ptr(w), _ptr(out), _i(dtype_code(x.dtype)), _i(M), _i(N), _i(K),
                                          _i(x.stride(0)), _i(w.stride(0)), _i(out.stride(0)), _i(epilogue), _stream())
    _check(st, "gemm_simt")
    return out


# --------------------------------------------------------------- rope + append
def rope_append(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, token_pos: torch.Tensor,
                token_seq: torch.Tensor, seq_slot: torch.Tensor, page_table: torch.Tensor,
                kpages: torch.Tensor, vpages: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                rotary_dim: int, interleaved: bool, write_cache: bool = True,
                parts: Optional[torch.Tensor] = None, clear_parts: bool = False) -> None:
    """Rotate q (in place) and k, and store k and v at their positions' pages.

    ``parts`` ([S, T, ld] fp32): the projection's unsummed K-slices; they are added here and ``qkv``
    only receives the rotated q.  ``clear_parts``: the kernel leaves zeros where it read
    ``parts`` (a sum that the projection adds into and that must be zero again for the next step)."""
    _need(qkv, None, "qkv")
    _need(cos, torch.float32, "cos")
    _need(sin, torch.float32, "sin")
    for n, t in (("token_pos", token_pos), ("token_seq", token_seq), ("seq_slot", seq_slot), ("page_table", page_table)):
        _need(t, torch.int32, n)
    _need(kpages, qkv.dtype, "kpages")
    _need(vpages, qkv.dtype, "vpages")
    T = qkv.shape[0]
    page_size = kpages.shape[-2]
    st = _lib("rope_append").dlgo_rope_append(
        _ptr(qkv), _i(dtype_code(qkv.dtype)), _i(T), _i(qkv.stride(0)), _ptr(cos), _ptr(sin), _ptr(token_pos),
        _ptr(token_seq), _ptr(seq_slot), _ptr(page_table), _i(page_table.shape[1]), _ptr(kpages), _ptr(vpages),
        _i(num_heads), _i(num_kv_heads), _i(head_dim), _i(rotary_dim), _i(page_size), _i(1 if interleaved else 0),
        _i(1 if write_cache else 0), _ptr(parts), _i(0 if parts is None else parts.shape[0]),
        _ll(0 if parts is None else parts.stride(0)), _i(1 if clear_parts else 0), _stream())
    _check(st, "rope_append")


# ------------------------------------------------------------------- attention
ATT_ROW_ELEMS = 128 * 32  # rows of a block times head_dim may not exceed this


def attention_tile_shape(head_dim: int, group: int, decode: bool) -> tuple[int, int]:
    """(tokens per tile, query heads of a kv head per block) that the kernel takes."""
    rows = max(1, ATT_ROW_ELEMS // head_dim)
    rows = min(rows, 32)
    gchunk = min(group, rows)
    qt = 1 if decode else max(1, min(8, rows // gchunk))
    return qt, gchunk


def attention_scratch_floats(T: int, num_heads: int, head_dim: int, n_splits: int) -> int:
    return 0 if n_splits <= 1 else T * num_heads * n_splits * (head_dim + 2)


def attention(q: torch.Tensor, ldq: int, T: int, kpages: torch.Tensor, vpages: torch.Tensor,
              page_table: torch.Tensor, tiles: torch.Tensor, tile_tokens_max: int, seq_slot: torch.Tensor,
              token_pos: torch.Tensor, out: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
              scale: float, window: int = 0, n_splits: int = 1, gchunk: int = 1,
              scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal grouped-query attention of T packed tokens over the paged cache."""
    _need(out, q.dtype, "out")
    _need(kpages, q.dtype, "kpages")
    _need(vpages, q.dtype, "vpages")
    for n, t in (("page_table", page_table), ("tiles", tiles), ("seq_slot", seq_slot), ("token_pos", token_pos)):
        _need(t, torch.int32, n)
    if n_splits > 1:
        need = attention_scratch_floats(T, num_heads, head_dim, n_splits)
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
            raise KernelError(f"attention: {n_splits} slices need {need} floats of scratch")
    st = _lib("attention").dlgo_attention(
        _ptr(q), _i(dtype_code(q.dtype)), _i(T), _i(ldq), _ptr(kpages), _ptr(vpages), _ptr(page_table),
        _i(page_table.shape[1]), _ptr(tiles), _i(tiles.shape[0]), _i(tile_tokens_max), _ptr(seq_slot),
        _ptr(token_pos), _ptr(out), _i(out.stride(0)), _ptr(scratch), _i(num_heads), _i(num_kv_heads), _i(head_dim),
        _i(kpages.shape[-2]), _i(n_splits), _i(gchunk), _i(window), _f(scale), _stream())
    _check(st, "attention", 2 if n_splits > 1 else 1)
    return out


# -------------------------------------------------------------------- sampling
def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """First index of each row's maximum (int32 on the device)."""
    _need(logits, torch.float32, "logits")
    R, V = logits.shape
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    _need(out, torch.int32, "out")
    lib = _lib("sampling")
    chunks = lib.dlgo_argmax_chunks(_i(R), _i(V))
    pv = pi = None
    if chunks > 1:
        pv = torch.empty((R * chunks,), dtype=torch.float32, device=logits.device)
        pi = torch.empty((R * chunks,), dtype=torch.int32, device=logits.device)
    st = lib.dlgo_argmax(_ptr(logits), _i(R), _i(logits.stride(0)), _i(V), _ptr(out), _ptr(pv), _ptr(pi), _stream())
    _check(st, "argmax", 2 if chunks > 1 else 1)
    return out


_argmax_host_buffers: dict = {}


def argmax_to_host(logits: torch.Tensor) -> list:
    """First index of each row's maximum, as a list of ints on the host: the kernels, the copy into a
    pinned buffer and the wait for it in one native call."""
    _need(logits, torch.float32, "logits")
    R, V = logits.shape
    key = (logits.device.index, R, V)
    buf = _argmax_host_buffers.get(key)
    lib = _lib("sampling")
    if buf is None:
        chunks = lib.dlgo_argmax_chunks(_i(R), _i(V))
        host = torch.zeros((R,), dtype=torch.int32).pin_memory()
        buf = _argmax_host_buffers[key] = (
            torch.empty((R,), dtype=torch.int32, device=logits.device),
            torch.empty((R * chunks,), dtype=torch.float32, device=logits.device) if chunks > 1 else None,
            torch.empty((R * chunks,), dtype=torch.int32, device=logits.device) if chunks > 1 else None,
            host, host.numpy(), 2 if chunks > 1 else 1)
    out, pv, pi, host, host_np, launches = buf
    st = lib.dlgo_argmax_host(_ptr(logits), _i(R), _i(logits.stride(0)), _i(V), _ptr(out), _ptr(pv), _ptr(pi),
                              _ptr(host), _stream())
    _check(st, "argmax", launches)
    return host_np.tolist()


def greedy_run_graph(host_inputs: torch.Tensor, graph_exec: int, host_ids: torch.Tensor,
                     stop_ids: Sequence[int], max_steps: int, device_index: int, launches_per_step: int) -> List[List[int]]:
    """Up to ``max_steps`` greedy decode steps of one batch in one native call (dlgo_greedy_run_graph).
    The captured step begins with the copy of its inputs out of ``host_inputs`` and ends with the argmax
    and the copy of the ids into ``host_ids`` (pinned int32 [B]);
    ``host_inputs`` (pinned int32 [3, B]: ids, positions, slots) holds the first step's inputs and is
    advanced in place.  Returns the ids chosen, a list per step, ending with the step in which a
    sequence chose a stop id."""
    import numpy as np
    B = host_ids.numel()
    stops = np.asarray(sorted(int(t) for t in stop_ids), dtype=np.int32)
    tokens = np.empty((max_steps, B), dtype=np.int32)
    n = _lib("sampling").dlgo_greedy_run_graph(
        ctypes.c_void_p(host_inputs.data_ptr()), _i(B), ctypes.c_void_p(graph_exec),
        ctypes.c_void_p(host_ids.data_ptr()), stops.ctypes.data_as(ctypes.c_void_p), _i(len(stops)), _i(max_steps),
        tokens.ctypes.data_as(ctypes.c_void_p), ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(device_index)))
    if n <= 0:
        raise KernelError(f"greedy_run_graph: error {n}")
    global LAUNCHES
    LAUNCHES += launches_per_step * n
    return tokens[:n].tolist()


def sampled_run_graph(host_inputs: torch.Tensor, graph_exec: int, host_ids: torch.Tensor, stop_ids: Sequence[int],
                      max_steps: int, draw_inputs: torch.Tensor, window: int, device_index: int,
                      launches_per_step: int) -> List[List[int]]:
    """:func:`greedy_run_graph` for sampled decoding (dlgo_sampled_run_graph): the captured step also copies
    ``draw_inputs`` (pinned int32: [2] seed, [B] requests, [B] draw indices, [B, window] recent tokens,
    [B] tokens produced so far) and ends with the filters and the draw; draw indices and windows are
    advanced in place."""
    import numpy as np
    B = host_ids.numel()
    if draw_inputs.numel() != 2 + 3 * B + B * window or draw_inputs.dtype != torch.int32 or not draw_inputs.is_pinned():
        raise KernelError("sampled_run_graph: draw_inputs must be pinned int32 [2 + 3 B + B window]")
    stops = np.asarray(sorted(int(t) for t in stop_ids), dtype=np.int32)
    tokens = np.empty((max_steps, B), dtype=np.int32)
    n = _lib("sampling").dlgo_sampled_run_graph(
        ctypes.c_void_p(host_inputs.data_ptr()), _i(B), ctypes.c_void_p(graph_exec),
        ctypes.c_void_p(host_ids.data_ptr()), stops.ctypes.data_as(ctypes.c_void_p), _i(len(stops)), _i(max_steps),
        tokens.ctypes.data_as(ctypes.c_void_p), ctypes.c_void_p(draw_inputs.data_ptr()), _i(window),
        ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(device_index)))
    if n <= 0:
        raise KernelError(f"sampled_run_graph: error {n}")
    global LAUNCHES
    LAUNCHES += launches_per_step * n
    return tokens[:n].tolist()


def sample(logits: torch.Tensor, temperature: torch.Tensor, request: torch.Tensor, draw: torch.Tensor, seed: int,
           out: Optional[torch.Tensor] = None, seed_dev: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row from softmax(logits / temperature) by inverse CDF; the uniform is a function of
    (seed, draw, request).  ``seed_dev`` (two int32 on the device, 8-byte aligned): the kernel reads the seed
    there instead (a captured step whose seed changes between replays)."""
    _need(logits, torch.float32, "logits")
    _need(temperature, torch.float32, "temperature")
    _need(request, torch.int32, "request")
    _need(draw, torch.int32, "draw")
    R, V = logits.shape
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    if seed_dev is not None and (seed_dev.dtype != torch.int32 or seed_dev.numel() < 2 or not seed_dev.is_cuda):
        raise KernelError("sample: seed_dev must be two int32 on the GPU")
    lib = _lib("sampling")
    chunks = int(lib.dlgo_sample_chunks(_i(V)))       # > 0: a large vocabulary, drawn from in two kernels
    part = torch.empty((R * chunks * 2,), dtype=torch.float32, device=logits.device) if chunks > 0 else None
    st = lib.dlgo_sample(_ptr(logits), _i(R), _i(logits.stride(0)), _i(V), _ptr(temperature), _ptr(request),
                         _ptr(draw), ctypes.c_ulonglong(seed & (2 ** 64 - 1)), _ptr(seed_dev), _ptr(out), _ptr(part),
                         _stream())
    _check(st, "sample", 2 if chunks > 0 else 1)
    return out


def uniform(seed: int, draw: torch.Tensor, request: torch.Tensor) -> torch.Tensor:
    _need(draw, torch.int32, "draw")
    _need(request, torch.int32, "request")
    out = torch.empty((draw.numel(),), dtype=torch.float32, device=draw.device)
    st = _lib("sampling").dlgo_uniform(ctypes.c_ulonglong(seed & (2 ** 64 - 1)), _ptr(draw), _ptr(request), _ptr(out),
                                       _i(draw.numel()), _stream())
    _check(st, "uniform")
    return out


# ------------------------------------------------------- tensor-core contraction
TC_STORE, TC_STORE_F32, TC_ADD_F32, TC_SWIGLU, TC_PARTIAL, TC_RED_F32 = 0, 1, 2, 3, 4, 5
TC_TILE_M, TC_TILE_K = 128, 64


def gemm_tc_workspace_floats(ra: int, rb: int, bn: int, splits: int) -> int:
    if splits <= 1:
        return 0
    return ((ra + TC_TILE_M - 1) // TC_TILE_M) * ((rb + bn - 1) // bn) * splits * bn * TC_TILE_M


def gemm_tc(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, transposed: bool, epilogue: int, bn: int,
            splits: int = 1, workspace: Optional[torch.Tensor] = None,
            counters: Optional[torch.Tensor] = None, static_operand: int = 0, pair_tile: int = 0) -> torch.Tensor:
    """D[Ra, Rb] = a[Ra, K] . b[Rb, K]^T on the tensor cores (bf16 in, fp32 accumulate).

    ``out`` receives D (``transposed``: D^T) through ``epilogue``; with ``splits`` > 1 the K range is
    shared by that many CTAs per tile, which needs ``workspace`` (fp32) and zeroed ``counters`` (int32).
    ``static_operand`` (1: a, 2: b) names the operand that holds weights no earlier kernel writes.
    ``pair_tile`` (128 or 256): many tokens, 256 x pair_tile tiles computed by pairs of CTAs (cta_group::2).
    ``TC_PARTIAL`` (transposed only): every K-slice leaves its fp32 tile in ``out`` [splits, Rb, Ra] for the
    reader to add in order.  ``TC_RED_F32`` (transposed only): every K-slice adds itself into the fp32
    ``out`` with reductions at the memory; no workspace, and the order of the adds (the sum's last bits) is
    not fixed.
    """
    if epilogue == TC_RED_F32 and not transposed:
        raise KernelError("gemm_tc: the atomic add is for transposed products")
    for n, t in (("a", a), ("b", b)):
        if not t.is_cuda or t.dtype != torch.bfloat16 or t.dim() != 2 or t.stride(1) != 1:
            raise KernelError(f"gemm_tc: {n} must be a 2-D bfloat16 GPU tensor with unit inner stride")
    ra, k = a.shape
    rb, k2 = b.shape
    if k != k2:
        raise KernelError(f"gemm_tc: a has K={k}, b has K={k2}")
    if out.stride(-1) != 1:
        raise KernelError("gemm_tc: out must have unit inner stride")
    if splits > 1 and epilogue not in (TC_PARTIAL, TC_RED_F32):
        need = gemm_tc_workspace_floats(ra, rb, bn, splits)
        tiles = ((ra + TC_TILE_M - 1) // TC_TILE_M) * ((rb + bn - 1) // bn)
        if workspace is None or workspace.numel() < need or counters is None or counters.numel() < tiles:
            raise KernelError(f"gemm_tc: {splits} K-slices need {need} floats of workspace and {tiles} counters")
    if epilogue == TC_PARTIAL:
        # out is [slices, rb, ra]: the kernel's row stride is that of one slice's rows
        if not transposed or out.dim() != 3 or out.dtype != torch.float32 or \
                tuple(out.shape) != (splits, rb, ra) or out.stride(0) != rb * out.stride(1) or out.stride(1) < ra:
            raise KernelError(f"gemm_tc: partials go to a float32 [{splits}, {rb}, {ra}] tensor of a transposed product")
        ldo = out.stride(1)
    else:
        want_shape = (rb, ra) if transposed else (ra, rb)
        if epilogue == TC_SWIGLU:
            want_shape = (rb, ra // 2) if transposed else (ra, rb // 2)
        if out.dim() != 2 or tuple(out.shape) != want_shape:
            raise KernelError(f"gemm_tc: out must be {list(want_shape)}, is {list(out.shape)}")
        want_dtype = torch.bfloat16 if epilogue in (TC_STORE, TC_SWIGLU) else torch.float32
        if out.dtype != want_dtype:
            raise KernelError(f"gemm_tc: out must be {want_dtype}")
        ldo = out.stride(0)
    st = _lib("gemm_tc").dlgo_gemm_tc(_ptr(a), _i(ra), _i(a.stride(0)), _ptr(b), _i(rb), _i(b.stride(0)), _i(k),
                                      _ptr(out), _i(ldo), _i(1 if transposed else 0), _i(epilogue), _i(bn),
                                      _i(splits), _ptr(workspace), _ptr(counters), _i(static_operand), _i(pair_tile),
                                      _stream())
    _check(st, "gemm_tc")
    return out


class RopeArgs(ctypes.Structure):
    """What the q|k|v projection's epilogue needs to rotate q and k and to append k and v (DlgoRopeArgs)."""
    _fields_ = [("cos_t", _p), ("sin_t", _p), ("token_pos", _p), ("token_seq", _p), ("seq_slot", _p),
                ("page_table", _p), ("max_pages", _i), ("kpages", _p), ("vpages", _p), ("Hq", _i), ("Hkv", _i),
                ("hd", _i), ("write_cache", _i)]


def rope_args(cos: torch.Tensor, sin: torch.Tensor, token_pos: torch.Tensor, token_seq: torch.Tensor,
              seq_slot: torch.Tensor, page_table: torch.Tensor, kpages: torch.Tensor, vpages: torch.Tensor,
              num_heads: int, num_kv_heads: int, head_dim: int, write_cache: bool) -> RopeArgs:
    """Checked :class:`RopeArgs`; the caller keeps the tensors alive while a launch may read them."""
    _need(cos, torch.float32, "cos")
    _need(sin, torch.float32, "sin")
    for n, t in (("token_pos", token_pos), ("token_seq", token_seq), ("seq_slot", seq_slot), ("page_table", page_table)):
        _need(t, torch.int32, n)
    _need(kpages, torch.bfloat16, "kpages")
    _need(vpages, torch.bfloat16, "vpages")
    if cos.dim() != 2 or cos.shape[1] * 2 != head_dim or sin.shape != cos.shape:
        raise KernelError("rope_args: whole-head rotation tables [positions, head_dim / 2] only")
    if kpages.shape[-2] != 64 or kpages.shape[-1] != head_dim or kpages.shape[-3] != num_kv_heads:
        raise KernelError("rope_args: pages must be [pages, kv heads, 64, head_dim]")
    return RopeArgs(cos.data_ptr(), sin.data_ptr(), token_pos.data_ptr(), token_seq.data_ptr(), seq_slot.data_ptr(),
                    page_table.data_ptr(), page_table.shape[1], kpages.data_ptr(), vpages.data_ptr(), num_heads,
                    num_kv_heads, head_dim, 1 if write_cache else 0)


def gemm_tc_rope_takes(out_features: int, in_features: int, num_heads: int, num_kv_heads: int, head_dim: int,
                       page_size: int) -> bool:
    """Whether :func:`gemm_tc_rope` takes a q|k|v weight [out, in] with these heads and pages."""
    import os
    return os.environ.get("DLGO_TC_DIRECT_EPILOGUE") is None and bool(_lib("gemm_tc").dlgo_gemm_tc_rope_takes(
        _i(out_features), _i(in_features), _i(num_heads), _i(num_kv_heads), _i(head_dim), _i(page_size)))


def gemm_tc_rope(x: torch.Tensor, w: torch.Tensor, qkv: torch.Tensor, pair_tile: int, rope: RopeArgs) -> torch.Tensor:
    """The q|k|v projection of a prompt step (``x`` [T, K] . ``w`` [(Hq + 2 Hkv) hd, K]^T on the tensor cores)
    whose epilogue rotates q and k in fp32 (whole head, split-half pairing), rounds once, writes the q heads to
    ``qkv`` [T, out] and appends k and v to the tokens' rows of their pages; the k and v columns of ``qkv`` are
    not written.  ``pair_tile``: 256 (CTA pairs) or 0."""
    for n, t in (("x", x), ("w", w)):
        if not t.is_cuda or t.dtype != torch.bfloat16 or t.dim() != 2 or t.stride(1) != 1:
            raise KernelError(f"gemm_tc_rope: {n} must be a 2-D bfloat16 GPU tensor with unit inner stride")
    T, k = x.shape
    n_out, k2 = w.shape
    if k != k2 or qkv.dtype != torch.bfloat16 or tuple(qkv.shape) != (T, n_out) or qkv.stride(1) != 1:
        raise KernelError("gemm_tc_rope: x [T, K], w [out, K] and a bfloat16 qkv [T, out] with unit inner stride")
    st = _lib("gemm_tc").dlgo_gemm_tc_rope(_ptr(x), _i(T), _i(x.stride(0)), _ptr(w), _i(n_out), _i(w.stride(0)), _i(k),
                                           _ptr(qkv), _i(qkv.stride(0)), _i(pair_tile), ctypes.byref(rope), _stream())
    _check(st, "gemm_tc_rope")
    return qkv


def check_device_errors() -> None:
    """Raise if a kernel gave up a bounded wait on the device since the last check (synchronises)."""
    for lib, fn in (("gemm_tc", "dlgo_gemm_tc_error"), ("attention_prefill_tc", "dlgo_attention_tc_error")):
        if lib in build._loaded:
            v = getattr(build._loaded[lib], fn)()
            if v != 0:
                raise KernelError(f"a tensor-core kernel ({lib}) gave up a bounded wait on the device; "
                                  "its results are invalid")
    if "decode_layers" in build._loaded:
        v = build._loaded["decode_layers"].dlgo_decode_layers_error()
        if v == 1:
            raise KernelError("the persistent decode kernel gave up a bounded wait on the device; its results are "
                              "invalid and its counters must be zeroed again (build a new engine)")
        if v != 0:
            raise KernelError("a token's position had no page in the cache's table (persistent decode kernel)")
    if "rope_append" in build._loaded and build._loaded["rope_append"].dlgo_rope_append_error() != 0:
        raise KernelError("a token's position had no page in the cache's table: its keys and values were not "
                          "stored and the step's results are invalid")


# ------------------------------------------------------------ decode attention
def attention_decode_mma_takes(dtype: torch.dtype, head_dim: int, page_size: int, n_splits: int) -> bool:
    """Whether the tensor-core decode kernel takes these sizes (bfloat16, heads of 64 or 128, 1..8 slices)."""
    return dtype == torch.bfloat16 and bool(
        _lib("attention_decode_mma").dlgo_attention_decode_mma_takes(_i(head_dim), _i(page_size), _i(n_splits)))


def attention_decode_mma_fuses_rope(num_heads: int, num_kv_heads: int, head_dim: int, rotary_dim: int,
                                    interleaved: bool) -> bool:
    """Whether the kernel can sum the projection's slices, rotate and append itself: whole-head rotation
    in the split-half pairing, at most 8 query heads per kv head."""
    return rotary_dim == head_dim and not interleaved and num_heads // num_kv_heads <= 8


def attention_decode_mma(q: Optional[torch.Tensor], ldq: int, B: int, kpages: torch.Tensor, vpages: torch.Tensor,
                         page_table: torch.Tensor, seq_slot: torch.Tensor, token_pos: torch.Tensor,
                         out: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                         window: int = 0, n_splits: int = 1, keys_per_tile: int = 16,
                         scratch: Optional[torch.Tensor] = None, parts: Optional[torch.Tensor] = None,
                         cos: Optional[torch.Tensor] = None, sin: Optional[torch.Tensor] = None,
                         write_cache: bool = True, clear_parts: bool = False) -> torch.Tensor:
    """Attention of one new token per sequence over its cached keys and values, bfloat16, on the
    tensor cores (mma.sync); 2..8 slices combine inside a thread-block cluster, more go through
    ``scratch`` (``attention_scratch_floats`` floats) and a second kernel.  With ``parts`` (the q|k|v
    projection as fp32 [slices, sequences, columns], unrotated) the kernel sums the slices, rotates q and k
    and appends k and v itself; ``clear_parts`` (one slice, at most 8 page slices): the sum is left zero."""
    for n, t in (("out", out), ("kpages", kpages), ("vpages", vpages)):
        _need(t, torch.bfloat16, n)
    for n, t in (("page_table", page_table), ("seq_slot", seq_slot), ("token_pos", token_pos)):
        _need(t, torch.int32, n)
    if seq_slot.numel() < B or token_pos.numel() < B or out.shape[0] < B:
        raise KernelError("attention_decode_mma: fewer rows than sequences")
    if out.shape[1] < num_heads * head_dim:
        raise KernelError("attention_decode_mma: out needs a column per head dimension")
    S = part_stride = 0
    if parts is None:
        _need(q, torch.bfloat16, "q")
        if q.shape[0] < B or q.shape[1] < num_heads * head_dim:
            raise KernelError("attention_decode_mma: q needs a row per sequence and a column per head dimension")
    else:
        # the projection's unsummed slices [S, B, ldq] (q | k | v heads), rotated and appended by the kernel
        _need(parts, torch.float32, "parts")
        _need(cos, torch.float32, "cos")
        _need(sin, torch.float32, "sin")
        if parts.dim() != 3 or parts.shape[1] < B or parts.shape[2] != ldq or \
                ldq < (num_heads + 2 * num_kv_heads) * head_dim or cos.shape[1] != head_dim // 2:
            raise KernelError("attention_decode_mma: parts must be [slices, sequences, q|k|v columns] with cos/sin "
                              "tables of head_dim / 2 columns")
        if not attention_decode_mma_fuses_rope(num_heads, num_kv_heads, head_dim, head_dim, False):
            raise KernelError("attention_decode_mma: these head counts cannot take the fused rotation")
        S, part_stride = parts.shape[0], parts.stride(0)
        if clear_parts and (S != 1 or n_splits > 8):
            raise KernelError("attention_decode_mma: only one summed slice read by at most 8 page slices can be cleared")
    if parts is None and clear_parts:
        raise KernelError("attention_decode_mma: clear_parts goes with parts")
    page_size = kpages.shape[-2]
    if n_splits > 8:
        need = attention_scratch_floats(B, num_heads, head_dim, n_splits)
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
            raise KernelError(f"attention_decode_mma: {n_splits} slices need {need} floats of scratch")
    st = _lib("attention_decode_mma").dlgo_attention_decode_mma(
        _ptr(q), _i(B), _i(ldq), _ptr(kpages), _ptr(vpages), _ptr(page_table), _i(page_table.shape[1]),
        _ptr(seq_slot), _ptr(token_pos), _ptr(out), _i(out.stride(0)), _i(num_heads), _i(num_kv_heads), _i(head_dim),
        _i(page_size), _i(n_splits), _i(window), _f(scale), _i(keys_per_tile),
        _ptr(scratch if n_splits > 8 else None), _ptr(parts), _i(S), _ll(part_stride), _ptr(cos), _ptr(sin),
        _i(1 if write_cache else 0), _i(1 if clear_parts else 0), _stream())
    _check(st, "attention_decode_mma", 2 if n_splits > 8 else 1)
    return out


def attention_decode_takes(dtype: torch.dtype, head_dim: int, page_size: int) -> bool:
    return bool(_lib("attention_decode").dlgo_attention_decode_takes(_i(dtype_code(dtype)), _i(head_dim), _i(page_size)))


def attention_decode(q: torch.Tensor, ldq: int, B: int, kpages: torch.Tensor, vpages: torch.Tensor,
                     page_table: torch.Tensor, seq_slot: torch.Tensor, token_pos: torch.Tensor, out: torch.Tensor,
                     num_heads: int, num_kv_heads: int, head_dim: int, scale: float, window: int = 0,
                     n_splits: int = 1, scratch: Optional[torch.Tensor] = None,
                     counters: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of one new token per sequence over its cached keys and values.

    ``counters`` (int32, zero, at least ``B * num_kv_heads * ceil(group / 4)``): with them the slice that
    finishes last combines the partial results; without them a second kernel does."""
    _need(out, q.dtype, "out")
    _need(kpages, q.dtype, "kpages")
    _need(vpages, q.dtype, "vpages")
    for n, t in (("page_table", page_table), ("seq_slot", seq_slot), ("token_pos", token_pos)):
        _need(t, torch.int32, n)
    if n_splits > 1 and not (scratch is None and n_splits <= 8):   # up to 8 slices can combine in a cluster
        need = attention_scratch_floats(B, num_heads, head_dim, n_splits)
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
            raise KernelError(f"attention_decode: {n_splits} slices need {need} floats of scratch")
        if counters is not None:
            _need(counters, torch.int32, "counters")
            if counters.numel() < B * num_kv_heads * ((num_heads // num_kv_heads + 3) // 4):
                raise KernelError("attention_decode: too few counters")
    st = _lib("attention_decode").dlgo_attention_decode(
        _ptr(q), _i(dtype_code(q.dtype)), _i(B), _i(ldq), _ptr(kpages), _ptr(vpages), _ptr(page_table),
        _i(page_table.shape[1]), _ptr(seq_slot), _ptr(token_pos), _ptr(out), _i(out.stride(0)), _ptr(scratch),
        _ptr(counters), _i(num_heads), _i(num_kv_heads), _i(head_dim), _i(kpages.shape[-2]), _i(n_splits), _i(window),
        _f(scale), _stream())
    _check(st, "attention_decode", 2 if (n_splits > 1 and counters is None and scratch is not None) else 1)
    return out


# ------------------------------------------------------ tensor-core prefill attention
PREFILL_TC_TILE = 128


def attention_prefill_tc_takes(dtype: torch.dtype, head_dim: int, page_size: int) -> bool:
    return dtype == torch.bfloat16 and head_dim in (64, 128) and page_size == 64


def attention_prefill_tc(q: torch.Tensor, ldq: int, T: int, kpages: torch.Tensor, vpages: torch.Tensor,
                         page_table: torch.Tensor, tiles: torch.Tensor, seq_slot: torch.Tensor,
                         token_pos: torch.Tensor, out: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                         scale: float, window: int = 0) -> torch.Tensor:
    """Causal attention of packed prompt tokens on the tensor cores; tiles hold at most 128 tokens each."""
    _need(out, torch.bfloat16, "out")
    _need(kpages, torch.bfloat16, "kpages")
    _need(vpages, torch.bfloat16, "vpages")
    if q.dtype != torch.bfloat16:
        raise KernelError("attention_prefill_tc: q must be bfloat16")
    for n, t in (("page_table", page_table), ("tiles", tiles), ("seq_slot", seq_slot), ("token_pos", token_pos)):
        _need(t, torch.int32, n)
    st = _lib("attention_prefill_tc").dlgo_attention_prefill_tc(
        _ptr(q), _i(T), _i(ldq), _ptr(kpages), _ptr(vpages), _i(kpages.shape[0]), _ptr(page_table),
        _i(page_table.shape[1]), _ptr(tiles), _i(tiles.shape[0]), _ptr(seq_slot), _ptr(token_pos), _ptr(out),
        _i(out.stride(0)), _i(num_heads), _i(num_kv_heads), _i(head_dim), _i(window), _f(scale), _stream())
    _check(st, "attention_prefill_tc")
    return out


# ------------------------------------------------------------------- filters
FILTER_MAX_K, FILTER_MAX_RECENT = 2048, 64


def filter_logits(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, min_p: float, penalty: float,
                  recent: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Repetition penalty, temperature, top-k (0: off, else up to 2048), top-p and min-p in one kernel.
    Returns the filtered, temperature-scaled logits; dropped tokens hold -inf.  ``recent`` is
    [rows, <= 64] int32 with -1 for "none"."""
    if not logits.is_cuda or logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("logits must be float32 [rows, vocab] on the GPU with unit stride along the vocabulary")
    R, V = logits.shape
    work = torch.empty((R, V), dtype=torch.float32, device=logits.device)
    n_recent = 0
    if recent is not None:
        _need(recent, torch.int32, "recent")
        n_recent = recent.shape[1]
    st = _lib("sampling").dlgo_filter(_ptr(logits), _i(R), _i(logits.stride(0)), _i(V), _ptr(work), _f(temperature),
                                      _i(top_k), _f(top_p), _f(min_p), _f(penalty), _ptr(recent), _i(n_recent),
                                      _stream())
    _check(st, "filter")
    return work


def filter_draw_chunks(V: int, top_k: int) -> int:
    """Chunks of the vocabulary :func:`filter_draw` works in, or 0 where it does not take the sizes (top-k off or
    above 256, a very large vocabulary): the caller then uses :func:`filter_logits` and :func:`sample`."""
    return int(_lib("sampling").dlgo_filter_draw_chunks(_i(V), _i(top_k)))


def filter_draw(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, min_p: float, penalty: float,
                recent: Optional[torch.Tensor], request: torch.Tensor, draw: torch.Tensor, seed: int,
                out: Optional[torch.Tensor] = None, seed_dev: Optional[torch.Tensor] = None) -> torch.Tensor:
    """:func:`filter_logits` followed by :func:`sample` for a small top-k, without a pass of one block over the
    whole row: blocks over chunks of the vocabulary list what top-k can keep, one block per row filters and
    draws from that list (csrc/sampling.cu)."""
    if not logits.is_cuda or logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("logits must be float32 [rows, vocab] on the GPU with unit stride along the vocabulary")
    R, V = logits.shape
    lib = _lib("sampling")
    C = int(lib.dlgo_filter_draw_chunks(_i(V), _i(top_k)))
    if C == 0:
        raise KernelError(f"filter_draw does not take top_k={top_k} with a vocabulary of {V}")
    cap = int(lib.dlgo_filter_draw_cap(_i(top_k)))
    _need(request, torch.int32, "request")
    _need(draw, torch.int32, "draw")
    n_recent = 0
    if recent is not None:
        _need(recent, torch.int32, "recent")
        n_recent = recent.shape[1]
    if seed_dev is not None and (seed_dev.dtype != torch.int32 or seed_dev.numel() < 2 or not seed_dev.is_cuda):
        raise KernelError("filter_draw: seed_dev must be two int32 on the GPU")
    dev = logits.device
    cand_v = torch.empty((R * C * cap,), dtype=torch.float32, device=dev)
    cand_i = torch.empty((R * C * cap + R * C,), dtype=torch.int32, device=dev)      # indices, then counts
    work = torch.empty((R, V), dtype=torch.float32, device=dev)      # (rows with more ties than the lists hold)
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=dev)
    st = lib.dlgo_filter_draw(_ptr(logits), _i(R), _i(logits.stride(0)), _i(V), _ptr(work), _f(temperature), _i(top_k),
                              _f(top_p), _f(min_p), _f(penalty), _ptr(recent), _i(n_recent), _ptr(cand_v),
                              _ptr(cand_i), _p(cand_i.data_ptr() + 4 * R * C * cap), _ptr(request), _ptr(draw),
                              ctypes.c_ulonglong(seed & (2 ** 64 - 1)), _ptr(seed_dev), _ptr(out), _stream())
    _check(st, "filter_draw", 2)
    return out


# ------------------------------------------------------------------ host side of a decode step
class HostStep:
    """The runtime calls of a decode step's launch as one native call: inputs out of a pinned buffer,
    an event that frees the buffer, the captured graph."""

    def __init__(self) -> None:
        lib = _lib("hoststep")
        lib.dlgo_hoststep_create.restype = ctypes.c_void_p
        self._lib = lib
        self._h = ctypes.c_void_p(lib.dlgo_hoststep_create())
        if not self._h:
            raise KernelError("hoststep: no event")

    def wait(self) -> None:
        st = self._lib.dlgo_hoststep_wait(self._h)
        if st != 0:
            raise KernelError(f"hoststep: CUDA error {st} while waiting for the input copy")

    def launch(self, dev_inputs: torch.Tensor, host_inputs: torch.Tensor, graph_exec: int, device_index: int) -> None:
        st = self._lib.dlgo_hoststep_launch(
            self._h, _ptr(dev_inputs), ctypes.c_void_p(host_inputs.data_ptr()),
            _ll(host_inputs.numel() * host_inputs.element_size()), ctypes.c_void_p(graph_exec),
            ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(device_index)))
        if st != 0:
            raise KernelError(f"hoststep: CUDA error {st} at the launch of a decode step")

    def __del__(self) -> None:
        try:
            self._lib.dlgo_hoststep_destroy(self._h)
        except Exception:
            pass


# ------------------------------------------------- a run of layers as one persistent kernel (decode steps)
def decode_layers_takes(tokens: int, hidden: int, num_heads: int, num_kv_heads: int, head_dim: int, ffn: int,
                        page_size: int) -> bool:
    """Whether the persistent decode kernel takes these sizes (see csrc/decode_layers.cu)."""
    return bool(_lib("decode_layers").dlgo_decode_layers_takes(_i(tokens), _i(hidden), _i(num_heads), _i(num_kv_heads),
                                                               _i(head_dim), _i(ffn), _i(page_size)))


def decode_layers_grid() -> int:
    return int(_lib("decode_layers").dlgo_decode_layers_grid())


def decode_layers_describe(layers: Sequence[dict], hidden: int, num_heads: int, num_kv_heads: int, head_dim: int,
                           ffn: int, device: torch.device) -> torch.Tensor:
    """The descriptor array of a run of layers, in device memory.  Each entry of ``layers`` gives the tensors
    ``w_qkv, w_o, w_gu, w_down`` (bfloat16, contiguous), ``norm1_w, norm2_w`` (float32), ``kpages, vpages``, and
    ``eps1, eps2, write_cache``.  The caller keeps those tensors alive as long as the descriptors are used."""
    lib = _lib("decode_layers")
    size = int(lib.dlgo_decode_layers_desc_bytes())
    raw = ctypes.create_string_buffer(size * len(layers) + 64)
    base = (ctypes.addressof(raw) + 63) & ~63
    for i, L in enumerate(layers):
        for n in ("w_qkv", "w_o", "w_gu", "w_down"):
            _need(L[n], torch.bfloat16, n)
        for n in ("norm1_w", "norm2_w"):
            _need(L[n], torch.float32, n)
        if L["kpages"].dtype != torch.bfloat16 or L["vpages"].dtype != torch.bfloat16:
            raise KernelError("decode_layers: the cache must be bfloat16")
        st = lib.dlgo_decode_layers_describe(
            ctypes.c_void_p(base + i * size), _ptr(L["w_qkv"]), _ptr(L["w_o"]), _ptr(L["w_gu"]), _ptr(L["w_down"]),
            _ptr(L["norm1_w"]), _ptr(L["norm2_w"]), _f(L["eps1"]), _f(L["eps2"]), _ptr(L["kpages"]), _ptr(L["vpages"]),
            _i(1 if L["write_cache"] else 0), _i(hidden), _i(num_heads), _i(num_kv_heads), _i(head_dim), _i(ffn))
        _check(st, "decode_layers_describe", 0)
    host = torch.frombuffer(bytearray(ctypes.string_at(base, size * len(layers))), dtype=torch.uint8)
    # device allocations are 256-byte aligned, which the tensor maps inside need
    return host.to(device)


def decode_layers_scratch_floats(tokens: int, num_heads: int, head_dim: int, n_splits: int) -> int:
    return int(_lib("decode_layers").dlgo_decode_layers_scratch_floats(_i(tokens), _i(num_heads), _i(head_dim),
                                                                         _i(n_splits)))


def decode_layers(desc: torch.Tensor, n_layers: int, residual: torch.Tensor, hidden: int, num_heads: int,
                  num_kv_heads: int, head_dim: int, ffn: int, scale: float, qkv_sum: torch.Tensor,
                  scale1: torch.Tensor, attn_out: torch.Tensor, h: torch.Tensor, scratch: Optional[torch.Tensor],
                  tickets: torch.Tensor, page_table: torch.Tensor, seq_slot: torch.Tensor, token_pos: torch.Tensor,
                  cos: torch.Tensor, sin: torch.Tensor, page_size: int, n_splits: int, sync: torch.Tensor,
                  first: bool = False) -> None:
    """``n_layers`` decoder layers on the residual stream [T, hidden] (fp32, in place), one new token per
    sequence: see csrc/decode_layers.cu.  ``qkv_sum``, ``tickets`` and ``sync`` must be zero and are left zero."""
    T = residual.shape[0]
    _need(residual, torch.float32, "residual")
    _need(qkv_sum, torch.float32, "qkv_sum")
    _need(scale1, torch.float32, "scale1")
    _need(attn_out, torch.bfloat16, "attn_out")
    _need(h, torch.bfloat16, "h")
    for n, t in (("tickets", tickets), ("page_table", page_table), ("seq_slot", seq_slot), ("token_pos", token_pos),
                 ("sync", sync)):
        _need(t, torch.int32, n)
    _need(cos, torch.float32, "cos")
    _need(sin, torch.float32, "sin")
    qkv_n = (num_heads + 2 * num_kv_heads) * head_dim
    if (residual.shape[1] != hidden or qkv_sum.numel() < T * qkv_n or scale1.numel() < T or
            attn_out.numel() < T * num_heads * head_dim or h.numel() < T * ffn or tickets.numel() < T * num_kv_heads or
            sync.numel() < 2 or seq_slot.numel() < T or token_pos.numel() < T):
        raise KernelError("decode_layers: a buffer is too small for these sizes")
    if cos.shape[1] * 2 != head_dim or sin.shape != cos.shape:
        raise KernelError("decode_layers: whole-head rotation tables [positions, head_dim / 2] only")
    if n_splits > 1:
        need = decode_layers_scratch_floats(T, num_heads, head_dim, n_splits)
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
            raise KernelError(f"decode_layers: {n_splits} page slices need {need} floats of scratch")
    st = _lib("decode_layers").dlgo_decode_layers(
        _ptr(desc), _i(n_layers), _i(T), _i(hidden), _i(num_heads), _i(num_kv_heads), _i(head_dim), _i(ffn), _f(scale),
        _ptr(residual), _i(residual.stride(0)), _ptr(qkv_sum), _ptr(scale1), _ptr(attn_out), _ptr(h), _ptr(scratch),
        _ptr(tickets), _ptr(page_table), _i(page_table.shape[1]), _ptr(seq_slot), _ptr(token_pos), _ptr(cos), _ptr(sin),
        _i(page_size), _i(n_splits), _i(0), _ptr(sync), _i(1 if first else 0), _stream())
    _check(st, "decode_layers")


# ------------------------------------------------------------------ the layer loop of a prompt step, native
class PromptEntryPoints(ctypes.Structure):
    _fields_ = [(n, _p) for n in ("rmsnorm", "gemm_tc", "rope_append", "attention", "gemm_tc_rope")]


class PromptShape(ctypes.Structure):
    _fields_ = [(n, _i) for n in ("hidden", "heads", "kv_heads", "head_dim", "ffn", "rotary_dim", "interleaved",
                                  "window", "page_size")] + [("scale", _f)]


class PromptLayer(ctypes.Structure):
    _fields_ = [("w_qkv", _p), ("w_o", _p), ("w_gate_up", _p), ("w_down", _p), ("norm1_w", _p), ("norm2_w", _p),
                ("eps1", _f), ("eps2", _f), ("kpages", _p), ("vpages", _p), ("n_pages", _i), ("write_cache", _i)]


class PromptStep(ctypes.Structure):
    _fields_ = [("tokens", _i), ("residual", _p), ("x", _p), ("qkv", _p), ("attn_out", _p), ("h", _p), ("cos_t", _p),
                ("sin_t", _p), ("token_pos", _p), ("token_seq", _p), ("seq_slot", _p), ("page_table", _p),
                ("max_pages", _i), ("tiles", _p), ("n_tiles", _i), ("bn", _i * 4), ("pair", _i * 4), ("fuse_rope", _i)]


PROMPT_CALLS = ("mixer norm", "q/k/v projection", "rotation and cache append (0 launches where the projection does it)", "attention", "output projection",
                "feed-forward norm", "gate/up projection", "down projection")


def prompt_entry_points() -> PromptEntryPoints:
    """Addresses of the entry points that the native layer loop calls (their libraries are loaded, and
    compiled first if need be)."""
    def address(lib: str, fn: str) -> int:
        return ctypes.cast(getattr(_lib(lib), fn), ctypes.c_void_p).value
    return PromptEntryPoints(address("elementwise", "dlgo_rmsnorm"), address("gemm_tc", "dlgo_gemm_tc"),
                             address("rope_append", "dlgo_rope_append"),
                             address("attention_prefill_tc", "dlgo_attention_prefill_tc"),
                             address("gemm_tc", "dlgo_gemm_tc_rope"))


def prompt_layers_describe(layers: Sequence[dict]) -> tuple:
    """The host-side descriptor array of a run of layers: (ctypes array, the tensors it points at, which the
    caller keeps alive with it).  Each entry gives ``w_qkv, w_o, w_gate_up, w_down`` (bfloat16, contiguous),
    ``norm1_w, norm2_w`` (float32), ``kpages, vpages`` (bfloat16) and ``eps1, eps2, write_cache``."""
    arr = (PromptLayer * len(layers))()
    keep = []
    for i, L in enumerate(layers):
        for n in ("w_qkv", "w_o", "w_gate_up", "w_down", "kpages", "vpages"):
            _need(L[n], torch.bfloat16, n)
        for n in ("norm1_w", "norm2_w"):
            _need(L[n], torch.float32, n)
        a = arr[i]
        for n in ("w_qkv", "w_o", "w_gate_up", "w_down", "norm1_w", "norm2_w", "kpages", "vpages"):
            setattr(a, n, L[n].data_ptr())
            keep.append(L[n])
        a.eps1, a.eps2 = L["eps1"], L["eps2"]
        a.n_pages, a.write_cache = L["kpages"].shape[0], 1 if L["write_cache"] else 0
    return arr, keep


def prompt_layers(entry: PromptEntryPoints, shape: PromptShape, layers: ctypes.Array, step: PromptStep) -> None:
    """Run ``len(layers)`` pre-norm layers of a prompt step: eight launches a layer (seven where the q/k/v
    projection rotates and appends in its epilogue: ``step.fuse_rope``), issued from one native loop
    (csrc/prompt_layers.cu).  The caller has checked types and sizes of what ``step`` points at."""
    failed = _i(-1)
    n = len(layers)
    st = _lib("prompt_layers").dlgo_prompt_layers(ctypes.byref(entry), ctypes.byref(shape), layers, _i(n),
                                                  ctypes.byref(step), ctypes.byref(failed), _stream())
    if st != 0 and failed.value >= 0:
        _check(st, f"prompt_layers (layer {failed.value // 8} of the run, {PROMPT_CALLS[failed.value % 8]})")
    _check(st, "prompt_layers", (7 if step.fuse_rope else 8) * n)
