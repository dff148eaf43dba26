"""The one-token step as a single persistent kernel, where the model allows it.

A decode step at small batch is a chain of short dependent kernels; `csrc/decode_stack.cu` runs
the whole chain (every schedule entry, the final norm and the head) in one launch whose blocks
stay resident and meet at grid-wide barriers. That kernel knows one arrangement of parts:
pre-norm blocks of RMSNorm, grouped-query attention with a fully rotated head over pages of 64
without a window, and a SwiGLU feed-forward, all in bfloat16 with the same sizes in every layer.
Whether a model is such a stack is asked of its parts (`stack_view()`), not of its architecture
name; a model with any other part, or a batch beyond the kernel's limit, runs part by part.
Measured slower than the CUDA graph of stand-alone kernels so far (1.21 ms against 0.77 ms per step
at the Llama 3.2 1B shape, batch 8), so it is used only when LLMIE_STACKED_DECODE=1 is set.
The reference captures the same step for batch 1 as a graph of its ~17 launches per layer
(src/cuda_graph.py:23-70).
"""
from __future__ import annotations

import os
import struct
from typing import List, Optional

import torch

from ..kernels import ops

MAX_LANES = 8


def _layer_view_ok(v: Optional[dict]) -> bool:
    return (v is not None and v["kind"] == "pre_norm" and v["mixer"]["kind"] == "gqa_rope"
            and v["feed_forward"]["kind"] == "swiglu" and v["mixer_norm"]["kind"] == "rmsnorm"
            and v["feed_forward_norm"]["kind"] == "rmsnorm")


class StackedDecode:
    """Built once per engine by `StackedDecode.plan(engine)`; None when the model is not such a stack."""

    @classmethod
    def plan(cls, engine) -> Optional["StackedDecode"]:
        if os.environ.get("LLMIE_STACKED_DECODE", "0") != "1" or engine.dtype != torch.bfloat16:
            return None
        model, cache = engine.model, engine.cache
        views = [model.blocks[call.layer].stack_view() for call in model.spec.schedule]
        final = model.final_norm.stack_view()
        if not views or not all(_layer_view_ok(v) for v in views) or final is None or final["kind"] != "rmsnorm":
            return None
        m0, f0 = views[0]["mixer"], views[0]["feed_forward"]
        d, ff = m0["hidden"], f0["intermediate"]
        n_q, n_kv, hd = m0["n_heads"], m0["n_kv_heads"], m0["head_dim"]
        for v in views:
            m, f = v["mixer"], v["feed_forward"]
            if (m["hidden"], m["n_heads"], m["n_kv_heads"], m["head_dim"]) != (d, n_q, n_kv, hd) \
                    or (f["hidden"], f["intermediate"]) != (d, ff):
                return None
            if any(w.dtype != torch.bfloat16 for w in (m["qkv"], m["o"], f["gate_up"], f["down"])):
                return None
        if model.embedding.dtype != torch.bfloat16 or model.head.weight.dtype != torch.bfloat16:
            return None
        if model.hidden_size != d or final["size"] != d:
            return None
        units = [cache.unit(model.unit_of_entry[pos]) for pos in range(len(views))]
        kv0 = units[0].kv
        for u in units:
            if u.kv is None or u.kv.block_table is not kv0.block_table or u.kv.page_size != 64 or u.kv.window \
                    or u.kv.k.dtype != torch.bfloat16:
                return None
        if not ops.decode_stack_supported(1, d, ff, n_q, n_kv, hd, model.vocab_size):
            return None
        return cls(engine, views, final, units)

    def __init__(self, engine, views: List[dict], final: dict, units):
        self.engine = engine
        model = engine.model
        dev = engine.device
        m0 = views[0]["mixer"]
        self.d, self.ff = m0["hidden"], views[0]["feed_forward"]["intermediate"]
        self.n_q, self.n_kv, self.hd = m0["n_heads"], m0["n_kv_heads"], m0["head_dim"]
        self.vocab = model.vocab_size
        self.n_layers = len(views)
        self.final_norm, self.final_eps = final["weight"], final["eps"]
        self.block_table = units[0].kv.block_table
        records = b""
        self._keep = []          # the tensors the table points into
        for pos, (v, u) in enumerate(zip(views, units)):
            m, f = v["mixer"], v["feed_forward"]
            owns = model.spec.schedule[pos].cache_of is None
            table = m["rope_table"]
            records += struct.pack(ops.STACK_LAYER_FORMAT, m["qkv"].data_ptr(), m["o"].data_ptr(),
                                   f["gate_up"].data_ptr(), f["down"].data_ptr(),
                                   v["mixer_norm"]["weight"].data_ptr(), v["feed_forward_norm"]["weight"].data_ptr(),
                                   u.kv.k.data_ptr(), u.kv.v.data_ptr(), table.data_ptr(),
                                   float(v["mixer_norm"]["eps"]), float(v["feed_forward_norm"]["eps"]),
                                   float(m["scale"]), int(table.shape[0]), 1 if owns else 0, 0)
            self._keep.append((v, u))
        if len(records) != self.n_layers * ops.decode_stack_layer_bytes():
            raise ops.KernelError("decode_stack: the layer record layout does not match the kernel's")
        self.layers = torch.frombuffer(bytearray(records), dtype=torch.uint8).to(dev)
        self.sync_words = torch.zeros(2, dtype=torch.int64, device=dev)
        self.counters = torch.zeros(8 * self.n_kv, dtype=torch.int32, device=dev)
        f32 = dict(dtype=torch.float32, device=dev)
        bf = dict(dtype=torch.bfloat16, device=dev)
        self.h = torch.zeros((MAX_LANES, self.d), **f32)
        self.q = torch.zeros((MAX_LANES, self.n_q * self.hd), **bf)
        self.attn = torch.zeros((MAX_LANES, self.n_q * self.hd), **bf)
        self.act = torch.zeros((MAX_LANES, self.ff), **bf)

    def supports(self, n_lanes: int) -> bool:
        return 1 <= n_lanes <= MAX_LANES

    def buffers(self, n_lanes: int, kv_limit: int):
        """Per captured step: partial results of attention for `kv_limit` positions, and the logits."""
        n_runs = (kv_limit + 63) // 64
        f32 = dict(dtype=torch.float32, device=self.engine.device)
        rows = n_lanes * self.n_q * n_runs
        return dict(n_runs=n_runs, part_m=torch.empty(rows, **f32), part_l=torch.empty(rows, **f32),
                    part_acc=torch.empty(rows * self.hd, **f32), logits=torch.empty((n_lanes, self.vocab), **f32))

    def run(self, tokens: torch.Tensor, slots: torch.Tensor, n_lanes: int, buf: dict,
            phase_ns: Optional[torch.Tensor] = None) -> torch.Tensor:
        e = self.engine
        ops.decode_stack(self.layers, self.n_layers, e.model.embedding, self.final_norm, self.final_eps,
                         e.model.head.weight, self.d, self.ff, self.n_q, self.n_kv, self.hd, tokens, slots,
                         e.cache.seq_lens, n_lanes, e.cache.scratch_slot, self.block_table, buf["n_runs"], self.h,
                         self.q, self.attn, self.act, buf["part_m"], buf["part_l"], buf["part_acc"], buf["logits"],
                         self.sync_words, self.counters, phase_ns)
        return buf["logits"]
