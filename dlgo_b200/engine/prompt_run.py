"""Runs of layers whose prompt step is issued from one native loop.

A prompt step of the usual pre-norm block (grouped-query attention with rotary
positions, SwiGLU feed-forward, RMSNorm) is eight launches a layer.  Issued one
by one from the parts' Python, they cost 19 us of host time each: 2.6 ms for 16
layers whatever the prompt's length, more than the GPU needs for 1,000 tokens.
Where consecutive run entries are such blocks with equal sizes, a prompt step
calls the same entry points with the same arguments from
``csrc/prompt_layers.cu`` instead.  This is a schedule, not a part: it reads
sizes, constants, tensors and tile shapes from the parts the model was built
from, launches what they launch, and steps aside (the parts run one by one) for
anything else: other blocks, mixers, feed-forwards or norms, float32, head
sizes the tensor-core attention does not take, few tokens, per-kernel timing.

``DLGO_NATIVE_PROMPT=0`` switches it off.
"""
from __future__ import annotations

import os
import weakref
from typing import Any, Dict, List, Optional

import torch

from ..csrc import kernels as K
from ..parts import tensor_core
from ..parts.attention import GQAAttention
from ..parts.block import PreNormBlock
from ..parts.feedforward import SwiGLU
from ..parts.norm import RMSNorm
from ..parts.rope import RotaryEmbedding

ENABLED = os.environ.get("DLGO_NATIVE_PROMPT", "1") != "0"


def _signature(blk: Any, positions: Dict[str, Any]) -> Optional[tuple]:
    """What two blocks must share to run in one native loop, or ``None`` if the loop does not take the block."""
    if type(blk) is not PreNormBlock:
        return None
    m, f, n1, n2 = blk.mixer, blk.ffn, blk.mixer_norm, blk.ffn_norm
    if type(m) is not GQAAttention or type(f) is not SwiGLU or type(n1) is not RMSNorm or type(n2) is not RMSNorm:
        return None
    if not getattr(f, "fused", False) or m.wqkv is None or m.wo is None:
        return None
    linears = (m.wqkv, m.wo, f.w_gate_up, f.w_down)
    if any(l.weight.dtype != torch.bfloat16 or getattr(l, "_tc", None) is None for l in linears):
        return None
    if n1.size != m.hidden_size or n2.size != m.hidden_size or n1.out_dtype != torch.bfloat16:
        return None
    rot, inter = 0, False
    if m.position_encoding is not None:
        pe = positions.get(m.position_encoding)
        if type(pe) is not RotaryEmbedding:
            return None
        rot, inter = pe.rotary_dim, pe.interleaved
    return (m.hidden_size, m.num_heads, m.num_kv_heads, m.head_dim, f.intermediate_size, m.scale, m.window or 0,
            m.position_encoding, rot, bool(inter), m.cache_group)


class PromptRun:
    """Run entries ``first .. first + n - 1`` of the model, issued by one native call per prompt step."""

    def __init__(self, first: int, n: int, sig: tuple):
        self.first, self.n, self.sig = first, n, sig
        self._layers: Dict[int, tuple] = {}       # per cache (its pages are part of the descriptors)
        self._entry: Optional[K.PromptEntryPoints] = None

    def takes(self, ctx: Any, cache: Any) -> bool:
        hd = self.sig[3]
        view = cache.view(self.first)
        return (not ctx.decode and ctx.n_tokens > tensor_core.SKINNY_MAX and view is not None and
                K._profile_events is None and
                K.attention_prefill_tc_takes(torch.bfloat16, hd, view.page_size) and view.keys.dtype == torch.bfloat16)

    def _descriptors(self, model: Any, cache: Any) -> tuple:
        hit = self._layers.get(id(cache))
        if hit is not None and hit[0]() is not cache:
            hit = None                          # another cache at a recycled address
        if hit is None:
            layers = []
            for i in range(self.first, self.first + self.n):
                blk = model.blocks[model.order[i].layer]
                view = cache.view(i)
                layers.append(dict(
                    w_qkv=blk.mixer.wqkv.weight, w_o=blk.mixer.wo.weight, w_gate_up=blk.ffn.w_gate_up.weight,
                    w_down=blk.ffn.w_down.weight, norm1_w=blk.mixer_norm.weight, norm2_w=blk.ffn_norm.weight,
                    eps1=blk.mixer_norm.eps, eps2=blk.ffn_norm.eps, kpages=view.keys, vpages=view.values,
                    write_cache=view.writes))
            hit = self._layers[id(cache)] = (weakref.ref(cache),) + K.prompt_layers_describe(layers)
        return hit[1], hit[2]

    def run(self, model: Any, residual: torch.Tensor, ctx: Any, cache: Any) -> None:
        d, hq, hkv, hd, f, scale, window, pe_name, rot, inter, _ = self.sig
        T = ctx.n_tokens
        view = cache.view(self.first)
        blk = model.blocks[model.order[self.first].layer]
        if residual.dtype != torch.float32 or not residual.is_contiguous() or tuple(residual.shape) != (T, d):
            raise K.KernelError("the residual stream must be contiguous float32 [tokens, hidden]")
        if self._entry is None:
            self._entry = K.prompt_entry_points()
        layers, _keep = self._descriptors(model, cache)
        if pe_name is not None:
            pe = model.positions[pe_name]
            cos, sin = pe.cos, pe.sin
        else:
            cos = sin = blk.mixer._no_rotation
        n_cols = (hq + 2 * hkv) * hd
        tiles, n_tiles, _ = ctx.tiles(K.PREFILL_TC_TILE, heaviest_first=True)
        step = K.PromptStep()
        step.tokens = T
        step.residual = residual.data_ptr()
        step.x = ctx.scratch("prompt_x", T * d, torch.bfloat16).data_ptr()
        step.qkv = ctx.scratch("prompt_qkv", T * n_cols, torch.bfloat16).data_ptr()
        step.attn_out = ctx.scratch("prompt_attn_out", T * hq * hd, torch.bfloat16).data_ptr()
        step.h = ctx.scratch("prompt_h", T * f, torch.bfloat16).data_ptr()
        step.cos_t, step.sin_t = cos.data_ptr(), sin.data_ptr()
        step.token_pos, step.token_seq = ctx.token_pos.data_ptr(), ctx.token_seq.data_ptr()
        step.seq_slot, step.page_table = ctx.seq_slot.data_ptr(), view.page_table.data_ptr()
        step.max_pages = view.page_table.shape[1]
        step.tiles, step.n_tiles = tiles.data_ptr(), n_tiles
        for j, lin in enumerate((blk.mixer.wqkv, blk.mixer.wo, blk.ffn.w_gate_up, blk.ffn.w_down)):
            step.bn[j], step.pair[j] = lin._tc.many_token_shape(T)
        step.fuse_rope = 1 if (pe_name is not None and blk.mixer.fuses_prompt_rope(ctx, view, model.positions)) else 0
        shape = K.PromptShape(d, hq, hkv, hd, f, rot, 1 if inter else 0, window, view.page_size, scale)
        K.prompt_layers(self._entry, shape, layers, step)


def plan_runs(model: Any, runtime: Any) -> Dict[int, PromptRun]:
    """{first run entry: PromptRun} for the model's runs of blocks the native loop takes (empty when switched
    off, in float32, or when no block qualifies)."""
    if not ENABLED or runtime.dtype != torch.bfloat16:
        return {}
    runs: Dict[int, PromptRun] = {}
    i, order = 0, model.order
    while i < len(order):
        sig = _signature(model.blocks[order[i].layer], model.positions)
        if sig is None:
            i += 1
            continue
        j = i + 1
        while j < len(order) and _signature(model.blocks[order[j].layer], model.positions) == sig:
            j += 1
        runs[i] = PromptRun(i, j - i, sig)
        i = j
    return runs
