"""Matrix products y = x W^T of the parts (no bias), chosen by the weight's precision.

bfloat16 weights: up to 8 rows this library's skinny kernel (up to 16 with the add, for up to one of its
blocks an SM); above that the library GEMM (cuBLAS through torch.mm), as the reference does with nn.Linear (src/model.py:17-19,34-37,137),
accumulating in float32, except where this library's weight-streaming tcgen05 kernel measured faster
(`ops.gemm_stream_wins`: a vocabulary-sized head at 33 to 64 rows). float32 weights: this
library's own FMA kernel, true 32-bit with a fixed summation order; that is the whole of
the 32-bit path, and also what a bfloat16 engine does with a tensor that its checkpoint
stores in 32-bit.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops


class Linear:
    def __init__(self, weight: torch.Tensor):
        if weight.dim() != 2:
            raise ValueError(f"a linear weight must be [out, in], got {tuple(weight.shape)}")
        if weight.dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"linear weight dtype {weight.dtype} is not supported")
        self.weight = weight.contiguous()
        self.out_features, self.in_features = weight.shape

    def nbytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def __call__(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """x [T, in] float32 or bfloat16 -> [T, out] in out_dtype (default: x's dtype)."""
        out_dtype = out_dtype or x.dtype
        w = self.weight
        if w.dtype == torch.float32:
            y = ops.gemm_f32_nt(x if x.dtype == torch.float32 else x.float(), w)
            return y if out_dtype == torch.float32 else y.to(out_dtype)
        xb = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
        T = xb.shape[0]
        if T <= ops.SKINNY_BEST_BATCH and ops.gemm_skinny_ok(T, self.out_features, self.in_features):
            f32 = out_dtype == torch.float32
            out = torch.empty((T, self.out_features), dtype=out_dtype, device=x.device)
            return ops.gemm_skinny(xb, w, out, ops.SKINNY_STORE_F32 if f32 else ops.SKINNY_STORE_BF16)
        if ops.gemm_stream_wins(T, self.out_features, self.in_features):
            out = torch.empty((T, self.out_features), dtype=out_dtype, device=x.device)
            return ops.gemm_stream(xb, w, out, ops.STREAM_STORE_F32 if out_dtype == torch.float32
                                   else ops.STREAM_STORE_BF16)
        return ops.library_mm(xb, w, out_dtype)

    def add_into(self, x: torch.Tensor, h: torch.Tensor) -> bool:
        """h (float32 [T, out]) += x W^T inside the product's kernel, when a kernel for this shape
        exists. Returns False (and does nothing) otherwise."""
        if self.weight.dtype != torch.bfloat16 or x.dtype != torch.bfloat16:
            return False
        if not ops.gemm_skinny_add_wins(x.shape[0], self.out_features, self.in_features, x.device) \
                or not ops.gemm_skinny_ok(x.shape[0], self.out_features, self.in_features):
            return False
        ops.gemm_skinny(x, self.weight, h, ops.SKINNY_ADD_F32)
        return True

    def swiglu(self, x: torch.Tensor) -> Optional[torch.Tensor]:
        """For a weight that is [gate rows; up rows]: silu(x Wg^T) * (x Wu^T) in one kernel, or None
        when no kernel for this shape exists."""
        if self.weight.dtype != torch.bfloat16 or x.dtype != torch.bfloat16:
            return None
        if x.shape[0] > ops.SKINNY_BEST_BATCH or not ops.gemm_skinny_ok(x.shape[0], self.out_features,
                                                                         self.in_features, ops.SKINNY_SWIGLU):
            return None
        out = torch.empty((x.shape[0], self.out_features // 2), dtype=torch.bfloat16, device=x.device)
        return ops.gemm_skinny(x, self.weight, out, ops.SKINNY_SWIGLU)
