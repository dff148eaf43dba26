"""Which kernel serves which call. The float32 engine uses the plain kernels throughout; the
bfloat16 engine swaps in the fast ones where their size limits are met and says no otherwise,
in which case the caller falls back to the plain kernel of the same math (never to a CPU or
library path)."""
from __future__ import annotations

import torch


class KernelPlan:
    def __init__(self, engine):
        self.engine = engine
        self.bf16 = engine.dtype == torch.bfloat16

    def attention(self, ctx, q, kv, out, n_q, n_kv, head_dim, scale, window) -> bool:
        """Returns True when a specialised kernel ran."""
        return False
