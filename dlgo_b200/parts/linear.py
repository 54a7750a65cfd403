"""A weight matrix ``[out, in]`` and its contraction ``y = x . W^T``.

The reference keeps matrices row-major ``[out x in]`` and computes one dot
product per output row (models/llm/model.go:64-80, blas/blas.go:152-196).  In
float32 the contraction runs on the fp32 pipes; in bfloat16 on the tensor cores
where the kernel takes the sizes, on the fp32 pipes (bfloat16 operands, fp32
sums) where it does not.
"""
from __future__ import annotations

from typing import Any, Optional

import torch

from ..csrc import kernels as K

STORE, STORE_F32, ADD_F32 = K.EPI_STORE, K.EPI_STORE_F32, K.EPI_ADD_F32


class Linear:
    """``fused_swiglu``: the weight holds gate and up rows in blocks of 16 + 16 and the contraction's
    epilogue writes ``silu(gate) * up`` ([T, out/2]); only the tensor-core kernel offers it
    (:attr:`fuses_swiglu` says whether this weight got it)."""

    def __init__(self, weight: torch.Tensor, runtime: Any, fused_swiglu: bool = False):
        self.weight = runtime.compute_copy(weight).contiguous()
        self.out_features, self.in_features = self.weight.shape
        self.runtime = runtime
        self._tc = None
        if self.weight.dtype == torch.bfloat16:
            from . import tensor_core
            self._tc = tensor_core.plan_for(self.weight, swiglu=fused_swiglu)
        self.fuses_swiglu = fused_swiglu and self._tc is not None
        if fused_swiglu and not self.fuses_swiglu:
            raise ValueError("this weight cannot take the fused SwiGLU epilogue")

    def __call__(self, x: torch.Tensor, epilogue: int = STORE, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self._tc is not None:
            return self._tc(x, epilogue, out)
        return K.gemm_simt(x, self.weight, epilogue, out)

    def rope_qkv_takes(self, tokens: int, num_heads: int, num_kv_heads: int, head_dim: int, page_size: int) -> bool:
        """Whether, for this many tokens, this weight can run as the q|k|v projection whose epilogue rotates q and
        k (whole head, split-half pairs) and appends k and v to the cache (tensor-core kernel, many tokens)."""
        if self._tc is None or self.fuses_swiglu:
            return False
        from . import tensor_core
        return (tokens > tensor_core.SKINNY_MAX and self._tc.many_token_shape(tokens)[0] == 256 and
                K.gemm_tc_rope_takes(self.out_features, self.in_features, num_heads, num_kv_heads, head_dim, page_size))

    def rope_qkv(self, x: torch.Tensor, rope: Any, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        return self._tc.rope_qkv(x, out, rope)

    def sums_slices_at_memory(self, tokens: int) -> bool:
        """Whether, for this many tokens, the add epilogue runs as several K-slices that add themselves
        into the target with reductions at the memory (the target may then be a plain zeroed sum)."""
        return self._tc is not None and not self.fuses_swiglu and self._tc.sums_slices_at_memory(tokens)

    def partials(self, x: torch.Tensor, single_ok: bool = True, for_residual: bool = False) -> Optional[torch.Tensor]:
        """The product as unsummed fp32 K-slices [slices, tokens, out] where the kernel offers that
        (few tokens on the tensor cores), else ``None``; also ``None`` for a single slice unless
        ``single_ok`` (a caller that wants the finished product in the activation type), and, with
        ``for_residual`` (the caller would leave the slices for the next norm to add to the residual
        stream), where the kernel would rather add its slices into the residual itself."""
        if self._tc is not None and not self.fuses_swiglu:
            return self._tc.partials(x, single_ok, for_residual)
        return None
