"""Grouped-query attention over the cache, with rotary positions.

Reference (models/llm/forward.go:207-290): q, k, v projections in one dispatch
(:224), rotation of every q and k head at the token's position (:246-252),
append to the cache (:257), per head ``softmax(q.k * scale)`` over positions
``0..pos`` and the weighted sum of values with kv head ``h / (Hq/Hkv)``
(:258-278), output projection (:286); the caller adds the result to the
residual (:163).  Prompts run the same steps over all their positions and read
keys and values back from the cache (models/llm/forward_batch.go:135-210).

Every constant is a parameter: head counts, head size, score scale, an optional
window (keys t > pos - window only), the name of the position encoding to use,
and the cache group the layer's keys and values belong to.
"""
from __future__ import annotations

import os
from typing import Any, Callable, Dict, Mapping, Optional

import torch

from ..csrc import kernels as K
from .base import CacheNeed, Mixer, ParamSpec, PositionEncoding
from .linear import ADD_F32, STORE, Linear
from .registry import MIXERS

_CLUSTER_MAX = int(os.environ.get("DLGO_ATTN_CLUSTER_MAX", 8))     # slices up to this many combine in a cluster
_MMA_KEYS = int(os.environ.get("DLGO_ATTN_MMA_KEYS", 32))    # keys per warp iteration of the tensor-core decode kernel (0: off)
# few tokens: the projection's K-slices meet in one fp32 sum (reductions at the memory) that is zero between steps
_QKV_SUM = int(os.environ.get("DLGO_ATTN_QKV_SUM", 1))
# ... which the tensor-core decode kernel reads itself: it rotates q and k, appends k and v and clears the sum, so
# the rotation needs no launch of its own.  Measured on a B200 (Llama 3.2 1B sizes): 0.789 -> 0.761 ms a step at
# batch 8, 1.31 -> 1.28 ms at batch 64.
_FUSE_ROPE = int(os.environ.get("DLGO_ATTN_FUSE_ROPE", 1))
_FUSE_ROPE_MAX_HEAD = 64
# prompts: the q|k|v projection's epilogue rotates and appends (0: the rotation kernel runs behind it)
_PROMPT_ROPE = int(os.environ.get("DLGO_PROMPT_ROPE", 1))


_DECODE_BLOCKS = int(os.environ.get("DLGO_ATTN_BLOCKS", 0))   # blocks wanted in flight for decode attention (0: as many as are resident)


def _sm_count(device: torch.device) -> int:
    from .tensor_core import sm_count
    return sm_count(device)


class GQAAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                 window: Optional[int] = None, position_encoding: Optional[str] = "rope",
                 cache_group: str = "full"):
        super().__init__(hidden_size=hidden_size, num_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=head_dim,
                         scale=scale, window=window, position_encoding=position_encoding, cache_group=cache_group)
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads ({num_heads}) must be a multiple of num_kv_heads ({num_kv_heads})")
        if head_dim % 16:
            raise ValueError(f"head_dim must be a multiple of 16, got {head_dim}")
        if window is not None and window <= 0:
            raise ValueError(f"window must be positive or None, got {window}")
        self.hidden_size = int(hidden_size)
        self.num_heads = int(num_heads)
        self.num_kv_heads = int(num_kv_heads)
        self.head_dim = int(head_dim)
        self.scale = float(scale)
        self.window = None if window is None else int(window)
        self.position_encoding = position_encoding
        self.cache_group = cache_group
        self.q_dim = self.num_heads * self.head_dim
        self.kv_dim = self.num_kv_heads * self.head_dim
        self.wqkv: Optional[Linear] = None
        self.wo: Optional[Linear] = None
        self._no_rotation: Optional[torch.Tensor] = None

    # --------------------------------------------------------------- declarations
    def param_specs(self) -> Dict[str, ParamSpec]:
        return {
            "q_proj.weight": ParamSpec((self.q_dim, self.hidden_size)),
            "k_proj.weight": ParamSpec((self.kv_dim, self.hidden_size)),
            "v_proj.weight": ParamSpec((self.kv_dim, self.hidden_size)),
            "o_proj.weight": ParamSpec((self.hidden_size, self.q_dim)),
        }

    def cache_need(self) -> CacheNeed:
        return CacheNeed(self.cache_group, self.num_kv_heads, self.head_dim, self.window)

    def load(self, get: Callable[[str], torch.Tensor], runtime: Any) -> None:
        # one fused projection: rows q | k | v (the reference splits a fused tensor
        # the other way round, models/llm/loader.go:267-279)
        parts = [runtime.compute_copy(get(n)) for n in ("q_proj.weight", "k_proj.weight", "v_proj.weight")]
        self.wqkv = Linear(torch.cat(parts, dim=0), runtime)
        self.wo = Linear(get("o_proj.weight"), runtime)
        self._no_rotation = torch.zeros((1, 1), dtype=torch.float32, device=runtime.device)

    # -------------------------------------------------------------------- forward
    def _decode_slices(self, ctx: Any, cache: Any, T: int, group: int, pages: int):
        """(page slices per sequence, scratch, counters) of the decode kernels: slices so that every SM has
        several blocks (whole waves: rounded down); 2..8 slices form a thread-block cluster and combine
        through distributed shared memory, more (one very long sequence alone) go through scratch memory."""
        # (as many blocks as are resident at once: four per SM, two for heads above 64, whose kernel takes twice
        # the registers; measured on a B200 at the layer sizes of Llama 3.2 3B, heads of 128, batch 8: 4 slices
        # in one wave 1.83 ms a step, 8 slices in two waves 2.04 ms)
        blocks = _DECODE_BLOCKS or (4 if self.head_dim <= 64 else 2) * _sm_count(cache.keys.device)
        base_blocks = T * self.num_kv_heads * ((group + 3) // 4)
        n_splits = max(1, min(pages, blocks // base_blocks))
        scratch = counters = None
        if n_splits > _CLUSTER_MAX and pages <= 64 and _CLUSTER_MAX > 1:
            n_splits = _CLUSTER_MAX
        if n_splits > _CLUSTER_MAX:
            scratch = ctx.scratch("attention", K.attention_scratch_floats(T, self.num_heads, self.head_dim, n_splits))
            counters = ctx.zeros("attention_counters", T * self.num_kv_heads * ((group + 3) // 4))
        return n_splits, scratch, counters

    def fuses_prompt_rope(self, ctx: Any, cache: Any, positions: Mapping[str, PositionEncoding]) -> bool:
        """Whether this step's q|k|v projection rotates and appends in its own epilogue: a prompt step in
        bfloat16 of more tokens than the few-token kernel takes, whole-head rotation in the split-half pairing,
        heads and pages the tensor-core kernel takes."""
        if ctx.decode or self.position_encoding is None or not _PROMPT_ROPE:
            return False
        pe = positions[self.position_encoding]
        return (pe.rotary_dim == self.head_dim and not pe.interleaved and cache.keys.dtype == torch.bfloat16 and
                self.wqkv.rope_qkv_takes(ctx.n_tokens, self.num_heads, self.num_kv_heads, self.head_dim,
                                         cache.page_size))

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: Any, cache: Any,
                state: Optional[torch.Tensor], positions: Mapping[str, PositionEncoding]) -> None:
        T = ctx.n_tokens
        group = self.num_heads // self.num_kv_heads
        if self.position_encoding is not None:
            pe = positions[self.position_encoding]
            cos, sin, rot, inter = pe.cos, pe.sin, pe.rotary_dim, pe.interleaved
        else:
            cos = sin = self._no_rotation
            rot, inter = 0, False
        act = self.wqkv.weight.dtype
        n_cols = self.q_dim + 2 * self.kv_dim
        longest = ctx.capacity if ctx.captured else ctx.max_len
        pages = max(1, (longest + cache.page_size - 1) // cache.page_size)
        decode_kernel = ctx.decode and K.attention_decode_takes(act, self.head_dim, cache.page_size)
        n_splits, scratch, counters = self._decode_slices(ctx, cache, T, group, pages) if decode_kernel else (1, None, None)
        # bfloat16, common head sizes, one token per sequence: scores and weighted sum on the tensor cores
        mma = (decode_kernel and _MMA_KEYS > 0 and
               K.attention_decode_mma_takes(act, self.head_dim, cache.page_size, n_splits))
        out = torch.empty((T, self.q_dim), dtype=act, device=x.device)
        qkv = None
        rotated = False
        if _QKV_SUM and self.wqkv.sums_slices_at_memory(T):
            # few tokens: the projection's K-slices add themselves, at the memory, into one fp32 sum that is zero
            # between steps; whoever rotates reads it once and leaves zeros behind
            qkv_sum = ctx.zeros(f"qkv_sum{n_cols}", T * n_cols, torch.float32)[:T * n_cols].view(1, T, n_cols)
            # (heads of 64 only: at 128 the kernel is at its register limit and the fused form measured 2 to 3 %
            # slower in a whole step at the layer sizes of Llama 3.2 3B and 3.1 8B, batch 8)
            fuse = (mma and _FUSE_ROPE and n_splits <= 8 and self.head_dim <= _FUSE_ROPE_MAX_HEAD and
                    K.attention_decode_mma_fuses_rope(self.num_heads, self.num_kv_heads, self.head_dim, rot, inter))
            self.wqkv(x, ADD_F32, qkv_sum[0])
            if fuse:
                # the decode kernel rotates, appends and clears itself: no launch for the rotation
                K.attention_decode_mma(None, n_cols, T, cache.keys, cache.values, cache.page_table, ctx.seq_slot,
                                       ctx.token_pos, out, self.num_heads, self.num_kv_heads, self.head_dim,
                                       self.scale, self.window or 0, n_splits, _MMA_KEYS, None, qkv_sum, cos, sin,
                                       cache.writes, clear_parts=True)
                rotated = True
            else:
                qkv = torch.empty((T, n_cols), dtype=x.dtype, device=x.device)
                K.rope_append(qkv, cos, sin, ctx.token_pos, ctx.token_seq, ctx.seq_slot, cache.page_table, cache.keys,
                              cache.values, self.num_heads, self.num_kv_heads, self.head_dim, rot, inter, cache.writes,
                              qkv_sum, True)
        elif self.fuses_prompt_rope(ctx, cache, positions):
            # prompts: the projection's epilogue rotates q and k and appends k and v (no launch for that, and
            # one rounding to bfloat16 instead of two)
            rope = K.rope_args(cos, sin, ctx.token_pos, ctx.token_seq, ctx.seq_slot, cache.page_table, cache.keys,
                               cache.values, self.num_heads, self.num_kv_heads, self.head_dim, cache.writes)
            qkv = self.wqkv.rope_qkv(x, rope)
        else:
            # ... or leaves its K-slices unsummed for the rotation to add in order; else the finished product
            qkv_parts = self.wqkv.partials(x, single_ok=False)
            qkv = (self.wqkv(x, STORE) if qkv_parts is None else
                   torch.empty((T, n_cols), dtype=x.dtype, device=x.device))
            K.rope_append(qkv, cos, sin, ctx.token_pos, ctx.token_seq, ctx.seq_slot, cache.page_table, cache.keys,
                          cache.values, self.num_heads, self.num_kv_heads, self.head_dim, rot, inter, cache.writes,
                          qkv_parts, False)
        if rotated:
            pass
        elif mma:
            K.attention_decode_mma(qkv, qkv.stride(0), T, cache.keys, cache.values, cache.page_table, ctx.seq_slot,
                                   ctx.token_pos, out, self.num_heads, self.num_kv_heads, self.head_dim, self.scale,
                                   self.window or 0, n_splits, _MMA_KEYS, scratch)
        elif decode_kernel:
            K.attention_decode(qkv, qkv.stride(0), T, cache.keys, cache.values, cache.page_table, ctx.seq_slot,
                               ctx.token_pos, out, self.num_heads, self.num_kv_heads, self.head_dim, self.scale,
                               self.window or 0, n_splits, scratch, counters)
        elif not ctx.decode and K.attention_prefill_tc_takes(qkv.dtype, self.head_dim, cache.page_size):
            # prompts: 128 query rows per CTA on the tensor cores
            tiles, n_tiles, _ = ctx.tiles(K.PREFILL_TC_TILE, heaviest_first=True)
            K.attention_prefill_tc(qkv, qkv.stride(0), T, cache.keys, cache.values, cache.page_table, tiles,
                                   ctx.seq_slot, ctx.token_pos, out, self.num_heads, self.num_kv_heads,
                                   self.head_dim, self.scale, self.window or 0)
        else:
            qt, gchunk = K.attention_tile_shape(self.head_dim, group, ctx.decode)
            tiles, n_tiles, tile_max = ctx.tiles(qt)
            n_gchunks = (group + gchunk - 1) // gchunk
            base_blocks = n_tiles * self.num_kv_heads * n_gchunks
            target = 2 * _sm_count(x.device)
            n_splits = max(1, min(pages, -(-target // base_blocks))) if ctx.decode else 1
            scratch = None
            if n_splits > 1:
                scratch = ctx.scratch("attention",
                                      K.attention_scratch_floats(T, self.num_heads, self.head_dim, n_splits))
            K.attention(qkv, qkv.stride(0), T, cache.keys, cache.values, cache.page_table, tiles, tile_max,
                        ctx.seq_slot, ctx.token_pos, out, self.num_heads, self.num_kv_heads, self.head_dim,
                        self.scale, self.window or 0, n_splits, gchunk, scratch)
        parts = self.wo.partials(out, for_residual=True) if hasattr(ctx, "defer") else None
        if parts is not None:
            ctx.defer(residual, parts)      # the next norm adds the slices to the residual
        else:
            self.wo(out, ADD_F32, residual)


MIXERS.register("gqa_attention", GQAAttention)
