"""Grouped-query attention over the paged cache.

q = x Wq^T, k = x Wk^T, v = x Wv^T without bias; q and k position-encoded; scores
q.k / sqrt(head_dim) over the keys a token may see, softmax in float32, times v; heads
concatenated in head order, then Wo (src/model.py:39-90 of the reference). Query head h reads
key/value head h // (n_heads / n_kv_heads) (src/flash_attn.py:92-94). The three projections are
one GEMM over row-concatenated weights.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..cache.cache import KVRequest
from ..kernels import ops, trace
from .base import AttentionOptions, DeferredNorm, Mixer, ParamSpec, build_part, register_mixer
from .linear import Linear


class GroupedQueryAttention(Mixer):
    """params: hidden, n_heads, n_kv_heads, head_dim, position (PartSpec of a position encoding),
    window (0 = every earlier key), scale (None = 1/sqrt(head_dim))."""

    adds_to_residual = True
    accepts_deferred_norm = True

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        self.hidden = int(params["hidden"])
        self.n_heads = int(params["n_heads"])
        self.n_kv_heads = int(params["n_kv_heads"])
        self.head_dim = int(params["head_dim"])
        self.window = int(params.get("window") or 0)
        if self.n_heads % self.n_kv_heads:
            raise ValueError(f"n_heads ({self.n_heads}) must be a multiple of n_kv_heads ({self.n_kv_heads})")
        if self.head_dim % 16 or self.head_dim > 256:
            raise ValueError(f"head_dim {self.head_dim} is not supported by the attention kernels "
                             "(multiples of 16 up to 256)")
        scale = params.get("scale")
        self.scale = float(scale) if scale is not None else self.head_dim ** -0.5
        self.options = AttentionOptions(scale=self.scale, window=self.window)
        self.position = build_part("position_encoding", params["position"], runtime)
        self.qkv: Linear = None
        self.o: Linear = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        hq, hkv, hd, d = self.n_heads, self.n_kv_heads, self.head_dim, self.hidden
        return {"q_proj.weight": ParamSpec((hq * hd, d)), "k_proj.weight": ParamSpec((hkv * hd, d)),
                "v_proj.weight": ParamSpec((hkv * hd, d)), "o_proj.weight": ParamSpec((d, hq * hd))}

    def load(self, tensors):
        ws = [tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]]
        dtype = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        self.qkv = Linear(torch.cat([w.to(dtype) for w in ws], dim=0))
        self.o = Linear(tensors["o_proj.weight"])

    def weight_bytes(self) -> int:
        return self.qkv.nbytes() + self.o.nbytes()

    def cache_requests(self):
        return [KVRequest(self.n_kv_heads, self.head_dim, self.window)]

    def forward(self, x, ctx, unit, owns_cache, residual=None):
        kv = unit.kv
        q = None
        trace.push("QKV_proj")
        if isinstance(x, DeferredNorm):
            table = getattr(self.position, "fused_table", lambda hd: None)(self.head_dim)
            w = self.qkv.weight
            if x.kind == "rmsnorm" and table is not None and w.dtype == torch.bfloat16 and kv.k.dtype == torch.bfloat16:
                # one-token steps: norm, the three projections, rotation and the cache write in one kernel
                q = torch.empty((x.shape[0], self.n_heads * self.head_dim), dtype=torch.bfloat16, device=w.device)
                ops.norm_qkv_rope(x.h, x.weight, x.eps, w, q, kv.k, kv.v, table, ctx.tok_pos, ctx.tok_seq,
                                  ctx.seq_slot, kv.block_table, kv.page_size, self.n_heads, self.n_kv_heads,
                                  self.head_dim, owns_cache)
            else:
                x = x.apply()
        attended = False
        if q is None:
            qkv = self.qkv(x)
            trace.pop()
            if ctx.decode:
                # one-token steps of more than 8 rows: rotation and cache write inside the attention kernel
                out = torch.empty((qkv.shape[0], self.n_heads * self.head_dim), dtype=qkv.dtype, device=qkv.device)
                trace.push("FlashDecode")
                table = getattr(self.position, "fused_table", lambda hd: None)(self.head_dim)
                attended = ctx.attention_with_rope(qkv, table, kv, out, self.n_heads, self.n_kv_heads, self.head_dim,
                                                   self.options, owns_cache)
                trace.pop()
            if not attended:
                trace.push("RoPE+KV_cache")
                q = self.position.encode_and_store(qkv, ctx, kv, self.n_heads, self.n_kv_heads, self.head_dim,
                                                   owns_cache)
                trace.pop()
        else:
            trace.pop()
        if not attended:
            out = torch.empty_like(q)
            trace.push("FlashDecode" if ctx.decode else "FlashAttn")
            ctx.attention(q, kv, out, self.n_heads, self.n_kv_heads, self.head_dim, self.options)
            trace.pop()
        trace.push("Output_proj")
        done = residual is not None and self.o.add_into(out, residual)
        y = None if done else self.o(out)
        trace.pop()
        return y


register_mixer("gqa_attention", GroupedQueryAttention)
