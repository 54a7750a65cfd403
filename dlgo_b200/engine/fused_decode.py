"""Runs of layers that a decode step hands to ONE persistent kernel.

A decode step of the usual pre-norm block (grouped-query attention with rotary
positions, SwiGLU feed-forward, RMSNorm) is eight small kernels a layer whose
hand-overs cost more than their work.  Where consecutive run entries are such
blocks with equal sizes, the step runs them as one launch of
``csrc/decode_layers.cu`` instead (bfloat16, at most 16 sequences).  This is a
schedule, not a part: it reads sizes, constants and tensors from the parts the
model was built from, computes what they compute, and steps aside (the parts
run one by one) for anything it does not take: other blocks, mixers,
feed-forwards or norms, windows, partial or interleaved rotation, other head
sizes, float32, more tokens.

Off by default (``DLGO_FUSED_DECODE=1`` switches it on): measured on a B200 at the
layer sizes of Llama 3.2 1B and batch 8, a layer takes 54 us in the persistent
kernel against 44 us as eight kernels chained by programmatic dependent launch.
Every phase ends in a grid-wide barrier (1.3 to 1.5 us each, five a layer) and
starts with a round trip to L2 for its operand that nothing overlaps, while the
separate kernels' prologues run under their predecessors' tails.
"""
from __future__ import annotations

import os
import weakref
from typing import Any, Dict, List, Optional

import torch

from ..csrc import kernels as K
from ..parts.attention import GQAAttention
from ..parts.block import PreNormBlock
from ..parts.feedforward import SwiGLU
from ..parts.norm import RMSNorm
from ..parts.rope import RotaryEmbedding

ENABLED = os.environ.get("DLGO_FUSED_DECODE", "0") == "1"
MAX_TOKENS = 16


def _signature(blk: Any, positions: Dict[str, Any]) -> Optional[tuple]:
    """What two blocks must share to run in one launch, or ``None`` if the kernel does not take the block."""
    if type(blk) is not PreNormBlock:
        return None
    m, f, n1, n2 = blk.mixer, blk.ffn, blk.mixer_norm, blk.ffn_norm
    if type(m) is not GQAAttention or type(f) is not SwiGLU or type(n1) is not RMSNorm or type(n2) is not RMSNorm:
        return None
    if m.window is not None or m.position_encoding is None or not getattr(f, "fused", False):
        return None
    pe = positions.get(m.position_encoding)
    if type(pe) is not RotaryEmbedding or pe.rotary_dim != m.head_dim or pe.interleaved:
        return None
    if m.wqkv is None or m.wqkv.weight.dtype != torch.bfloat16 or m.num_heads // m.num_kv_heads > 8:
        return None
    if m.head_dim not in (64, 128) or n1.size != m.hidden_size or n2.size != m.hidden_size:
        return None
    return (m.hidden_size, m.num_heads, m.num_kv_heads, m.head_dim, f.intermediate_size, m.scale, m.position_encoding,
            m.cache_group)


class FusedRun:
    """Run entries ``first .. first + n - 1`` of the model as one launch per decode step."""

    def __init__(self, first: int, entries: List[int], sig: tuple):
        self.first, self.entries, self.sig = first, entries, sig
        self.n = len(entries)
        self._desc: Dict[int, tuple] = {}      # per cache (its pages are part of the descriptors)

    def takes(self, ctx: Any, cache: Any) -> bool:
        d, hq, hkv, hd, f = self.sig[:5]
        view = cache.view(self.first)
        return (ctx.decode and ctx.n_tokens <= MAX_TOKENS and view is not None and
                K.decode_layers_takes(ctx.n_tokens, d, hq, hkv, hd, f, view.page_size))

    def _descriptors(self, model: Any, cache: Any, device: torch.device) -> torch.Tensor:
        hit = self._desc.get(id(cache))
        if hit is not None and hit[0]() is not cache:
            hit = None                          # another cache at a recycled address
        if hit is None:
            d, hq, hkv, hd, f = self.sig[:5]
            layers = []
            for i in range(self.first, self.first + self.n):
                blk = model.blocks[model.order[i].layer]
                view = cache.view(i)
                layers.append(dict(
                    w_qkv=blk.mixer.wqkv.weight, w_o=blk.mixer.wo.weight, w_gu=blk.ffn.w_gate_up.weight,
                    w_down=blk.ffn.w_down.weight, norm1_w=blk.mixer_norm.weight, norm2_w=blk.ffn_norm.weight,
                    eps1=blk.mixer_norm.eps, eps2=blk.ffn_norm.eps, kpages=view.keys, vpages=view.values,
                    write_cache=view.writes))
            hit = self._desc[id(cache)] = (weakref.ref(cache), K.decode_layers_describe(layers, d, hq, hkv, hd, f, device))
        return hit[1]

    def run(self, model: Any, residual: torch.Tensor, ctx: Any, cache: Any) -> None:
        d, hq, hkv, hd, f, scale, pe_name, _ = self.sig
        T = ctx.n_tokens
        view = cache.view(self.first)
        pe = model.positions[pe_name]
        desc = self._descriptors(model, cache, residual.device)
        longest = ctx.capacity if ctx.captured else ctx.max_len
        pages = max(1, (longest + view.page_size - 1) // view.page_size)
        n_splits = max(1, min(pages, K.decode_layers_grid() // (T * hkv)))
        qkv_n = (hq + 2 * hkv) * hd
        qkv_sum = ctx.zeros(f"fused_qkv_sum{qkv_n}", T * qkv_n, torch.float32)
        tickets = ctx.zeros("fused_tickets", T * hkv)
        sync = ctx.zeros("fused_sync", 2)
        scale1 = ctx.scratch("fused_scale1", T)
        attn_out = ctx.scratch("fused_attn_out", T * hq * hd, torch.bfloat16)
        h = ctx.scratch("fused_h", T * f, torch.bfloat16)
        scratch = None
        if n_splits > 1:
            scratch = ctx.scratch("attention", K.decode_layers_scratch_floats(T, hq, hd, n_splits))
        K.decode_layers(desc, self.n, residual, d, hq, hkv, hd, f, scale, qkv_sum, scale1, attn_out, h, scratch,
                        tickets, view.page_table, ctx.seq_slot, ctx.token_pos, pe.cos, pe.sin, view.page_size, n_splits,
                        sync)


def plan_runs(model: Any, runtime: Any) -> Dict[int, FusedRun]:
    """{first run entry: FusedRun} for the model's runs of blocks the kernel takes (empty when switched off,
    in float32, or when no block qualifies)."""
    from ..parts import tensor_core
    if not ENABLED or runtime.dtype != torch.bfloat16 or tensor_core.ORDERED_SUMS:
        return {}
    runs: Dict[int, FusedRun] = {}
    i, order = 0, model.order
    while i < len(order):
        sig = _signature(model.blocks[order[i].layer], model.positions)
        if sig is None:
            i += 1
            continue
        j = i + 1
        while j < len(order) and _signature(model.blocks[order[j].layer], model.positions) == sig:
            j += 1
        runs[i] = FusedRun(i, list(range(i, j)), sig)
        i = j
    return runs
