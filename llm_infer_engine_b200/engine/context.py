"""What one step looks like to the parts: the ragged batch as device index arrays plus the
host-side bounds needed to size launches, and the attention service that picks a kernel.

    tokens     [T]    token ids of all sequences, packed one sequence after another
    tok_pos    [T]    absolute position of each token in its sequence
    tok_seq    [T]    which sequence of this step (0..n-1) each token belongs to
    cu_q       [n+1]  where each sequence's tokens start in the packed arrays
    seq_slot   [n]    cache slot of each sequence
    seq_start  [n]    tokens the sequence held before this step
    seq_kvlen  [n]    tokens it holds after this step
    logit_rows [R]    packed rows whose logits are wanted
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..kernels import ops
from ..parts.base import AttentionOptions


@dataclass
class StepContext:
    n_tokens: int
    n_seqs: int
    decode: bool                 # every sequence brings exactly one token
    max_q_len: int               # host-side upper bounds, for launch sizing only
    max_kv_len: int
    tokens: torch.Tensor
    tok_pos: torch.Tensor
    tok_seq: torch.Tensor
    cu_q: torch.Tensor
    seq_slot: torch.Tensor
    seq_start: torch.Tensor
    seq_kvlen: torch.Tensor
    logit_rows: torch.Tensor
    dtype: torch.dtype
    device: torch.device
    kernels: Optional[object] = None     # the engine's kernel choices (KernelPlan)
    all_rows: bool = False               # logit_rows is 0..n_tokens-1: every row's logits are wanted
    entry: int = 0                       # which entry of the run order is running (set by the model, for traces)

    def attention_with_rope(self, qkv, table, kv, out, n_q: int, n_kv: int, head_dim: int, options: AttentionOptions,
                            write_kv: bool) -> bool:
        """Attention straight from the packed projections `qkv` of a one-token step, with the rotation by
        `table` (a whole-head (cos, sin) table) and the cache write inside the attention kernel. Returns False
        when no kernel does that for this step; the caller then encodes and stores first and calls `attention`."""
        plan = self.kernels
        return plan is not None and plan.attention_with_rope(self, qkv, table, kv, out, n_q, n_kv, head_dim, options,
                                                             write_kv)

    def attention(self, q, kv, out, n_q: int, n_kv: int, head_dim: int, options: AttentionOptions) -> None:
        """softmax(q k^T * scale) v over the cache unit `kv`, each token seeing the keys of its own
        sequence up to its own position (and no further back than `options.window`, if set)."""
        plan = self.kernels
        if plan is not None and plan.attention(self, q, kv, out, n_q, n_kv, head_dim, options):
            return
        ops.attention_paged(q, kv.k, kv.v, out, self.tok_pos, self.tok_seq, self.seq_slot, kv.block_table,
                            kv.page_size, n_q, n_kv, head_dim, options.scale, options.window)
