"""Which kernel serves which call. The float32 engine uses the plain kernels throughout; the
bfloat16 engine swaps in the fast ones where their size limits are met and says no otherwise,
in which case the caller falls back to the plain kernel of the same math (never to a CPU or
library path)."""
from __future__ import annotations

import torch

from ..kernels import ops


class KernelPlan:
    MIN_COUNTERS = 4096            # counters allocated at least; more than any one-token step of 64 lanes needs

    def __init__(self, engine):
        self.engine = engine
        self.bf16 = engine.dtype == torch.bfloat16
        self._counters = None          # zeroed once; the decode attention kernel leaves them zero
        self._retired = []             # outgrown counter tensors that captured steps may still point to
        self.decode_attention = engine.decode_attention      # "auto", or "split": always the CUDA-core kernel

    def _decode_counters(self, need: int, device) -> torch.Tensor:
        """Zeroed counters for the merge of a decode attention launch. A captured step keeps the address
        it was captured with, so a tensor that has been handed out is never freed: when a later step needs
        more, the smaller tensor stays alive beside the new one."""
        if self._counters is None or self._counters.numel() < need:
            if self._counters is not None:
                self._retired.append(self._counters)
            self._counters = torch.zeros(max(need, self.MIN_COUNTERS), dtype=torch.int32, device=device)
        return self._counters

    @staticmethod
    def decode_run_length(n_seqs: int, head_dim: int, dtype) -> int:
        """Keys per block of the split-KV kernel: one cache page; the reference uses runs of 256
        (src/flash_decode.py:271-272). Depends only on the step's shape, never on its data."""
        return ops.attention_decode_run_len(n_seqs, head_dim, dtype)

    def attention_with_rope(self, ctx, qkv, table, kv, out, n_q, n_kv, head_dim, options, write_kv) -> bool:
        """One-token steps whose projections were not made by the fused norm + QKV kernel (more than 8 rows):
        rotation of q and k and the cache write happen inside the attention kernel, where a kernel for this
        size exists. Returns False (and does nothing) otherwise; the caller then rotates and stores first."""
        if not write_kv:
            return False       # a borrowed cache already holds the owner's new key: it must be read, not replaced
        if not (ctx.decode and self.decode_attention != "split" and qkv.dtype == torch.bfloat16
                and table is not None and ops.attention_decode_mma_supported(head_dim, qkv.dtype, kv.page_size)):
            return False
        pages = ops.attention_decode_mma_pages(ctx.n_seqs, n_q, n_kv, ctx.max_kv_len)
        n_runs = ((ctx.max_kv_len + 63) // 64 + pages - 1) // pages
        counters = self._decode_counters(ops.decode_counter_ints(ctx.n_seqs, n_q, n_kv), qkv.device)
        ops.attention_decode_mma_rope(qkv, kv.k, kv.v, out, table, ctx.seq_slot, ctx.seq_kvlen, kv.block_table,
                                      kv.page_size, n_q, n_kv, head_dim, options.scale, options.window, pages, n_runs,
                                      write_kv, counters=counters)
        return True

    def attention(self, ctx, q, kv, out, n_q, n_kv, head_dim, options) -> bool:
        """Returns True when a specialised kernel ran. Every kernel below takes the options there are
        today (scale, window); a new option is checked here, kernel by kernel."""
        scale, window = options.scale, options.window
        if ctx.decode and self.decode_attention != "split" \
                and ops.attention_decode_mma_supported(head_dim, q.dtype, kv.page_size):
            # bfloat16, head size 64 or 128: a warp per page on the tensor cores
            pages = ops.attention_decode_mma_pages(ctx.n_seqs, n_q, n_kv, ctx.max_kv_len)
            n_runs = ((ctx.max_kv_len + 63) // 64 + pages - 1) // pages
            counters = self._decode_counters(ops.decode_counter_ints(ctx.n_seqs, n_q, n_kv), q.device)
            ops.attention_decode_mma(q, kv.k, kv.v, out, ctx.seq_slot, ctx.seq_kvlen, kv.block_table, kv.page_size,
                                     n_q, n_kv, head_dim, scale, window, pages, n_runs, counters=counters)
            return True
        if ctx.decode and kv.page_size == 64 and ops.attention_decode_supported(head_dim, q.dtype):
            run = self.decode_run_length(ctx.n_seqs, head_dim, q.dtype)
            n_runs = (ctx.max_kv_len + run - 1) // run
            counters = self._decode_counters(ops.decode_counter_ints(ctx.n_seqs, n_q, n_kv), q.device)
            ops.attention_decode(q, kv.k, kv.v, out, ctx.seq_slot, ctx.seq_kvlen, kv.block_table, kv.page_size,
                                 n_q, n_kv, head_dim, scale, window, run, n_runs, counters=counters)
            return True
        if not ctx.decode and scale > 0 and ops.attention_prefill_tc_supported(head_dim, kv.page_size, q.dtype):
            ops.attention_prefill_tc(q, kv.k, kv.v, out, ctx.cu_q, ctx.seq_slot, ctx.seq_start, kv.block_table,
                                     kv.page_size, ctx.n_seqs, ctx.max_q_len, n_q, n_kv, head_dim, scale, window)
            return True
        return False
