"""Choice of the tensor-core contraction for a bfloat16 weight.

``plan_for(weight)`` returns a callable ``(x, epilogue, out) -> out`` that runs the tcgen05
kernel, or ``None`` when the kernel does not take the weight's sizes (the caller then uses the
fp32-pipe kernel, never a wrong result).

Few tokens (decode): the WEIGHT is the tensor core's M operand (128 rows per tile) and the tokens
are its N (16 / 32 / 64); tiles are written transposed, and the K range is shared by several CTAs
per tile so that every SM streams its part of the weight.  Many tokens: the activations are M, the
weight is N (tiles of 128 x 256), written row-major.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional

import os

import torch

from ..csrc import kernels as K

SKINNY_MAX = 64          # tokens up to which the weight is the M operand
# CTAs that share a weight: one per SM.  A CTA's ring takes under half an SM's shared memory, so the
# CTAs of the NEXT contraction move in beside it and fetch their first weights while this one still
# streams.  Two per SM would need more K-slices per tile, and every extra slice writes and re-reads a
# partial result of tokens x outputs floats (at 64 tokens half of the weight's own bytes) and makes
# the consumer's sum longer.  Measured on a B200 (tokens a second, 148 against 296 CTAs): 8.95K
# against 8.77K at batch 8, 35.2K against 30.3K at batch 64.
TARGET_CTAS = int(os.environ.get("DLGO_TC_TARGET_CTAS", 0))          # 0: the device's SM count
# At most 16 tokens a partial tile is small (and, where it goes into the residual, is added there with
# reductions at the memory and never read again): three CTAs per two SMs then stream better than one per
# SM.  Measured (tokens a second, 148 / 222 / 296): 9.90K / 10.10K / 10.05K at batch 8, 1.32K / 1.40K /
# 1.38K at batch 1; at batch 64, with tiles four times as wide, 49.0K / 42.9K / 39.7K.
TARGET_CTAS_FEW = int(os.environ.get("DLGO_TC_TARGET_CTAS_FEW", 0))  # 0: one and a half times the SM count
# ... and two per SM for a weight of 25 MB and more, whose K-slices are then still long (down at every size, q/k/v
# and o_proj at the larger ones).  Measured (ms a step at batch 8, three against four CTAs per two SMs for those
# weights): 0.760 -> 0.747 at Llama 3.2 1B sizes (0.698 -> 0.686 at batch 1), 1.827 -> 1.789 at 3B, 1.709 ->
# 1.645 at 8B; for every weight (threshold 0) 3B loses what it gained.  The SwiGLU product keeps one CTA per tile.
BIG_WEIGHT_BYTES = int(os.environ.get("DLGO_TC_BIG_WEIGHT_MB", 25)) << 20
MAX_SPLITS = int(os.environ.get("DLGO_TC_MAX_SPLITS", 32))    # upper bound on K-slices per tile
PAIR_TILE = int(os.environ.get("DLGO_TC_PAIR_TILE", 256))    # 0 switches the CTA-pair kernel off
PAIR_MIN_TOKENS = int(os.environ.get("DLGO_TC_PAIR_MIN_TOKENS", 64))   # CTA pairs for more tokens than this
MIN_KBLOCKS_PER_SPLIT = int(os.environ.get("DLGO_TC_MIN_KBLOCKS", 3))   # (3 against 4: 0.747 -> 0.742 ms at batch 8, 0.686 -> 0.680 at batch 1)
# Few tokens: a contraction whose result goes into the residual stream adds its K-slices there with
# reductions at the memory (up to RED_MAX_TOKENS tokens) instead of leaving them for the norm's kernel to
# add.  Measured on a B200 (Llama 3.2 1B sizes, tokens a second): 8.99K -> 9.90K at batch 8, 1.19K -> 1.32K at
# batch 1, 45.8K -> 49.0K at batch 64.  The order of such adds is not fixed, so the sums' last bits differ from
# run to run; DLGO_ORDERED_SUMS=1 keeps the K-slices apart and lets the next norm add them in slice order
# instead: slower, and bit for bit repeatable.
ORDERED_SUMS = os.environ.get("DLGO_ORDERED_SUMS", "0") == "1"
RED_MAX_TOKENS = int(os.environ.get("DLGO_TC_RED_MAX_TOKENS", 64))

_workspaces: Dict[int, List[torch.Tensor]] = {}
_counters: Dict[int, torch.Tensor] = {}


def _workspace(device: torch.device, floats: int) -> torch.Tensor:
    """One workspace per device, shared by all contractions (they run one after another on a stream).
    Buffers that were outgrown stay alive: a captured graph may still point at them."""
    lst = _workspaces.setdefault(device.index or 0, [])
    if not lst or lst[-1].numel() < floats:
        lst.append(torch.empty((max(floats, 1 << 20),), dtype=torch.float32, device=device))
    return lst[-1]


def _counter_buffer(device: torch.device) -> torch.Tensor:
    c = _counters.get(device.index or 0)
    if c is None:
        c = _counters[device.index or 0] = torch.zeros((1 << 16,), dtype=torch.int32, device=device)
    return c


_sm_counts: Dict[int, int] = {}


def sm_count(device: Optional[torch.device] = None) -> int:
    """SMs of the device (asked once per device)."""
    idx = torch.cuda.current_device() if device is None or device.index is None else device.index
    n = _sm_counts.get(idx)
    if n is None:
        n = _sm_counts[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return n


def skinny_shape(tokens: int, n: int, k: int, device: Optional[torch.device] = None,
                 fused_epilogue: bool = False) -> tuple[int, int]:
    """(bn, splits) for ``tokens`` <= SKINNY_MAX against a weight [n, k]; ``fused_epilogue``: the product's
    epilogue is not a plain sum (SwiGLU), so K-slices would have to meet in a workspace first."""
    bn = 16 if tokens <= 16 else (32 if tokens <= 32 else 64)
    tiles = (n + K.TC_TILE_M - 1) // K.TC_TILE_M
    kblocks = (k + K.TC_TILE_K - 1) // K.TC_TILE_K
    if tokens <= 16:
        big = n * k * 2 >= BIG_WEIGHT_BYTES and not fused_epilogue
        few = 2 * sm_count(device) if big else (3 * sm_count(device)) // 2
        target = TARGET_CTAS_FEW or few
    else:
        target = TARGET_CTAS or sm_count(device)
    splits = max(1, min(kblocks // MIN_KBLOCKS_PER_SPLIT, target // tiles)) if tiles < target else 1
    return bn, max(1, min(splits, kblocks, MAX_SPLITS))


class TensorCorePlan:
    def __init__(self, weight: torch.Tensor, swiglu: bool = False):
        self.weight = weight
        self.n, self.k = weight.shape
        self.swiglu = swiglu

    def __call__(self, x, epilogue: int, out: Optional[torch.Tensor]) -> torch.Tensor:
        t = x.shape[0]
        if self.swiglu:
            epi = K.TC_SWIGLU
            if out is None:
                out = torch.empty((t, self.n // 2), dtype=torch.bfloat16, device=x.device)
        else:
            epi = {K.EPI_STORE: K.TC_STORE, K.EPI_STORE_F32: K.TC_STORE_F32, K.EPI_ADD_F32: K.TC_ADD_F32}[epilogue]
            if out is None:
                if epilogue == K.EPI_ADD_F32:
                    raise K.KernelError("the add epilogue needs the tensor to add into")
                out = torch.empty((t, self.n), dtype=torch.bfloat16 if epilogue == K.EPI_STORE else torch.float32,
                                  device=x.device)
        if t <= SKINNY_MAX:
            bn, splits = skinny_shape(t, self.n, self.k, self.weight.device, self.swiglu)
            if not ORDERED_SUMS and epi == K.TC_ADD_F32 and splits > 1 and t <= RED_MAX_TOKENS:
                return K.gemm_tc(self.weight, x, out, True, K.TC_RED_F32, bn, splits, static_operand=1)
            ws = cnt = None
            if splits > 1:
                ws = _workspace(x.device, K.gemm_tc_workspace_floats(self.n, t, bn, splits))
                cnt = _counter_buffer(x.device)
            return K.gemm_tc(self.weight, x, out, True, epi, bn, splits, ws, cnt, static_operand=1)
        bn, pair = self.many_token_shape(t)
        return K.gemm_tc(x, self.weight, out, False, epi, bn, static_operand=2, pair_tile=pair)

    def many_token_shape(self, tokens: int) -> tuple[int, int]:
        """(tile width, CTA-pair tile or 0) for more than SKINNY_MAX tokens: the activations are the M operand."""
        bn = 256 if self.n > 128 else 128
        pair = PAIR_TILE if (tokens > PAIR_MIN_TOKENS and self.n >= 256) else 0      # CTA pairs share 256 x 256 tiles
        return bn, pair

    def rope_qkv(self, x, out: Optional[torch.Tensor], rope: "K.RopeArgs") -> torch.Tensor:
        """This weight as the q|k|v projection of a prompt step, its epilogue rotating q and k and appending k
        and v (``rope``: :func:`kernels.rope_args`); more than SKINNY_MAX tokens."""
        t = x.shape[0]
        if out is None:
            out = torch.empty((t, self.n), dtype=torch.bfloat16, device=x.device)
        bn, pair = self.many_token_shape(t)
        return K.gemm_tc_rope(x, self.weight, out, pair, rope)

    def sums_slices_at_memory(self, tokens: int) -> bool:
        if ORDERED_SUMS or tokens > min(RED_MAX_TOKENS, SKINNY_MAX):
            return False
        return skinny_shape(tokens, self.n, self.k, self.weight.device)[1] > 1

    def partials(self, x, single_ok: bool = True, for_residual: bool = False) -> Optional[torch.Tensor]:
        """For few tokens: the product's K-slices, unsummed, as fp32 [slices, tokens, out]; whoever
        reads the result next adds them in order (this spares the contraction a reduction pass through
        memory).  ``None`` when the tokens are too many for that, or, unless ``single_ok``, when there would be
        one slice only (the caller then asks for the finished product in the type it wants), or, with
        ``for_residual``, when the add epilogue would add the slices into the residual by itself."""
        t = x.shape[0]
        if t > SKINNY_MAX or self.swiglu:
            return None
        if for_residual and not ORDERED_SUMS and t <= RED_MAX_TOKENS:
            return None                     # the caller's add epilogue adds the slices into the residual
        bn, splits = skinny_shape(t, self.n, self.k, self.weight.device)
        if splits == 1 and not single_ok:
            return None
        out = torch.empty((splits, t, self.n), dtype=torch.float32, device=x.device)
        K.gemm_tc(self.weight, x, out, True, K.TC_PARTIAL, bn, splits, static_operand=1)
        return out


def plan_for(weight: torch.Tensor, swiglu: bool = False) -> Optional[Callable]:
    n, k = weight.shape
    if weight.dtype != torch.bfloat16 or k % 8 or weight.stride(1) != 1 or weight.stride(0) % 8:
        return None
    if weight.data_ptr() % 16:
        return None
    if swiglu and n % 32:
        return None
    return TensorCorePlan(weight, swiglu)
