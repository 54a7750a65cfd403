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

_TARGET_BLOCKS = 2 * 148  # blocks wanted in flight for decode attention (general kernel)
# The decode kernel can also rotate q and k and append k and v itself (one launch less per layer); measured
# inside a whole step it is no faster than the separate rope kernel, so it is opt-in: DLGO_ATTN_FUSE_ROPE=1.
_NO_FUSE = not os.environ.get("DLGO_ATTN_FUSE_ROPE")
_CLUSTER_MAX = int(os.environ.get("DLGO_ATTN_CLUSTER_MAX", 8))     # slices up to this many combine in a cluster
# keys and values that the rope kernel hints into L2 for the attention kernel, per layer (0: off, the
# default: measured on a B200 the hint does not pay, the attention kernel's own hint is early enough)
_AHEAD_BYTES = int(os.environ.get("DLGO_ATTN_AHEAD_MB", 0)) << 20
_MMA_KEYS = int(os.environ.get("DLGO_ATTN_MMA_KEYS", 32))    # keys per warp iteration of the tensor-core decode kernel (0: off)
# ... which can also sum the projection's slices, rotate and append itself (one launch less per layer).  Opt-in:
# measured in a whole step it is slower (0.918 against 0.891 ms at batch 8): every slice of a sequence repeats
# the sum of the query's K-slices, and the block that appends starts its keys a round trip later.
_QKV_SUM = int(os.environ.get("DLGO_ATTN_QKV_SUM", 1))   # the projection's K-slices meet in one fp32 sum
_MMA_FUSE = os.environ.get("DLGO_ATTN_MMA_FUSE_ROPE", "0") == "1"
_DECODE_BLOCKS = int(os.environ.get("DLGO_ATTN_BLOCKS", 4 * 148))  # and for the decode kernel, whose blocks are small


class GQAAttention(Mixer):
    takes_deferred_norm = True   # its first contraction may compute the norm of the residual itself

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
        decode_kernel = ctx.decode and K.attention_decode_takes(act, self.head_dim, cache.page_size)
        fused_rope = decode_kernel and not _NO_FUSE and K.attention_decode_fuses_rope(
            act, self.num_heads, self.num_kv_heads, self.head_dim, rot, inter, cache.page_size)
        # few tokens: the projection leaves its K-slices unsummed and whoever rotates adds them
        qkv = None
        clear_parts = False
        if _QKV_SUM and self.wqkv.sums_slices_at_memory(T) and not (fused_rope or _MMA_FUSE):
            # ... or its K-slices add themselves, at the memory, into one fp32 sum that is zero between
            # steps: the rotation reads it once and leaves zeros behind
            n = self.q_dim + 2 * self.kv_dim
            qkv_parts = ctx.zeros(f"qkv_sum{n}", T * n, torch.float32)[:T * n].view(1, T, n)
            self.wqkv(x, ADD_F32, qkv_parts[0])
            clear_parts = True
        else:
            qkv_parts = self.wqkv.partials(x, single_ok=False)
        if qkv_parts is None:
            qkv = self.wqkv(x, STORE)
        # the tensor-core decode kernel can take the slices as they are: it sums, rotates and appends itself
        mma_fused = (decode_kernel and _MMA_FUSE and _MMA_KEYS and qkv_parts is not None and not fused_rope and
                     K.attention_decode_mma_takes(act, self.head_dim, cache.page_size, 1) and
                     K.attention_decode_mma_fuses_rope(self.num_heads, self.num_kv_heads, self.head_dim, rot, inter))
        if not fused_rope and not mma_fused:
            if qkv is None:
                qkv = torch.empty((T, self.q_dim + 2 * self.kv_dim), dtype=x.dtype, device=x.device)
            ahead = 0
            if decode_kernel and qkv_parts is not None and _AHEAD_BYTES > 0:
                # pages of keys and values per (sequence, kv head) to hint into L2 for the attention kernel
                page_bytes = cache.page_size * self.head_dim * self.wqkv.weight.element_size()
                ahead = max(1, _AHEAD_BYTES // (2 * T * self.num_kv_heads * page_bytes))
            K.rope_append(qkv, cos, sin, ctx.token_pos, ctx.token_seq, ctx.seq_slot, cache.page_table, cache.keys,
                          cache.values, self.num_heads, self.num_kv_heads, self.head_dim, rot, inter, cache.writes,
                          qkv_parts, ahead, self.window or 0, clear_parts)
        longest = ctx.capacity if ctx.captured else ctx.max_len
        pages = max(1, (longest + cache.page_size - 1) // cache.page_size)
        out = torch.empty((T, self.q_dim), dtype=act, device=x.device)
        if decode_kernel:
            # one token per sequence: the latency-shaped kernel, sliced so that every SM has several blocks
            base_blocks = T * self.num_kv_heads * ((group + 3) // 4)
            n_splits = max(1, min(pages, _DECODE_BLOCKS // base_blocks))   # whole waves: rounded down
            scratch = counters = None
            if n_splits > _CLUSTER_MAX and pages <= 64 and _CLUSTER_MAX > 1:
                n_splits = _CLUSTER_MAX
            if n_splits > _CLUSTER_MAX:
                # very long sequences at small batches: slices through scratch, the last one combines
                scratch = ctx.scratch("attention",
                                      K.attention_scratch_floats(T, self.num_heads, self.head_dim, n_splits))
                counters = ctx.zeros("attention_counters", T * self.num_kv_heads * ((group + 3) // 4))
            # (2..8 slices form a thread-block cluster and combine through distributed shared memory)
            if mma_fused:
                K.attention_decode_mma(None, qkv_parts.shape[2], T, cache.keys, cache.values, cache.page_table,
                                       ctx.seq_slot, ctx.token_pos, out, self.num_heads, self.num_kv_heads,
                                       self.head_dim, self.scale, self.window or 0, n_splits, _MMA_KEYS, scratch,
                                       qkv_parts, cos, sin, cache.writes)
            elif (not fused_rope and _MMA_KEYS and
                    K.attention_decode_mma_takes(act, self.head_dim, cache.page_size, n_splits)):
                # bfloat16, common head sizes: the scores and the weighted sum on the tensor cores
                K.attention_decode_mma(qkv, qkv.stride(0), T, cache.keys, cache.values, cache.page_table,
                                       ctx.seq_slot, ctx.token_pos, out, self.num_heads, self.num_kv_heads,
                                       self.head_dim, self.scale, self.window or 0, n_splits, _MMA_KEYS, scratch)
            elif fused_rope:
                # rotation of q and k and the append of k and v happen inside the attention kernel
                K.attention_decode_rope(qkv, qkv_parts, T, cos, sin, rot, inter, cache.writes, cache.keys,
                                        cache.values, cache.page_table, ctx.seq_slot, ctx.token_pos, out,
                                        self.num_heads, self.num_kv_heads, self.head_dim, self.scale,
                                        self.window or 0, n_splits, scratch, counters)
            else:
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
            n_splits = max(1, min(pages, -(-_TARGET_BLOCKS // base_blocks))) if ctx.decode else 1
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
