"""Dense gated feed-forward: down(silu(gate x) * (up x)), no bias (src/model.py:14-25 of the
reference, w1 = gate, w3 = up, w2 = down). gate and up are one GEMM over row-concatenated
weights; the activation and product are one kernel."""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels import ops, trace
from .base import DeferredNorm, FeedForward, ParamSpec, register_feed_forward
from .linear import Linear


class SwiGLU(FeedForward):
    """params: hidden, intermediate."""

    adds_to_residual = True
    accepts_deferred_norm = True

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        self.hidden = int(params["hidden"])
        self.intermediate = int(params["intermediate"])
        self.gate_up: Linear = None
        self.down: Linear = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"gate_proj.weight": ParamSpec((self.intermediate, self.hidden)),
                "up_proj.weight": ParamSpec((self.intermediate, self.hidden)),
                "down_proj.weight": ParamSpec((self.hidden, self.intermediate))}

    def load(self, tensors):
        g, u = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        dtype = torch.float32 if torch.float32 in (g.dtype, u.dtype) else g.dtype
        self.gate_up = Linear(torch.cat([g.to(dtype), u.to(dtype)], dim=0))
        self.down = Linear(tensors["down_proj.weight"])

    def weight_bytes(self) -> int:
        return self.gate_up.nbytes() + self.down.nbytes()

    def forward(self, x, ctx, residual=None):
        trace.push("FFN")
        try:
            return self._forward(x, ctx, residual)
        finally:
            trace.pop()

    def _forward(self, x, ctx, residual):
        act = None
        if isinstance(x, DeferredNorm):
            w = self.gate_up.weight
            if x.kind == "rmsnorm" and w.dtype == torch.bfloat16 and self.intermediate % 8 == 0:
                # one-token steps: norm, product, activation and gate in one kernel
                act = torch.empty((x.shape[0], self.intermediate), dtype=torch.bfloat16, device=w.device)
                ops.norm_gate_swiglu(x.h, x.weight, x.eps, w, act)
            else:
                x = x.apply()
        if act is None:
            act = self.gate_up.swiglu(x)             # product, activation and gate in one kernel
        if act is None:
            gu = self.gate_up(x)
            act = torch.empty((x.shape[0], self.intermediate), dtype=gu.dtype, device=x.device)
            ops.swiglu(gu, act)
        if residual is not None and self.down.add_into(act, residual):
            return None
        return self.down(act)


register_feed_forward("swiglu", SwiGLU)
