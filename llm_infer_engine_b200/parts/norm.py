"""RMSNorm fused with the residual add that precedes it.

y = x * rsqrt(mean(x^2) + eps) * w, all in float32, one rounding at the store
(src/rms_norm.py:32-39 of the reference). The weight is used as it is (not 1 + w).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops, trace
from .base import DeferredNorm, Norm, ParamSpec, register_norm


class RMSNorm(Norm):
    """params: size (width of a row), eps."""

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.size,), role="vector", init=tuple(self.params.get("init", ("ones",))))}

    def load(self, tensors):
        self.weight = tensors["weight"].to(torch.float32).contiguous()   # bf16 -> f32 is exact

    def weight_bytes(self) -> int:
        return self.size * 4

    def defer(self, h):
        """One-token steps of the bfloat16 engine: the next product's kernel applies this norm itself."""
        if self.runtime.dtype != torch.bfloat16 or not ops.norm_gemm_supported(h.shape[0], self.size):
            return None
        return DeferredNorm(self, h, "rmsnorm", self.weight, self.eps)

    def forward(self, h, delta, out=None, rows=None):
        n_out = h.shape[0] if rows is None else rows.shape[0]
        if out is None:
            out = torch.empty((n_out, self.size), dtype=self.runtime.dtype, device=h.device)
        trace.push("RMSNorm")
        ops.add_rmsnorm(h, delta, self.weight, self.eps, out, rows)
        trace.pop()
        return out


register_norm("rmsnorm", RMSNorm)
