"""Rotary position encoding (rotate-half pairing) with optional llama3 frequency scaling.

Frequencies: inv_i = theta^(-2i/rot_dim), i < rot_dim/2 (src/rope.py:9 of the reference); the
llama3 rule rescales them by wavelength (src/rope.py:11-30). Angles p * inv_i, their cosines
and sines are float32 (src/rope.py:35-37). The reference then rounds cos and sin to the
activation dtype and rotates in it (src/rope.py:43-44,75-86); here the table stays float32 and
the rotation is done in float32 in both precisions. Rotation is fused with the cache write
(src/rope.py:122-185): keys are stored rotated.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..kernels import ops
from .base import PositionEncoding, register_position_encoding


def inverse_frequencies(rot_dim: int, theta: float, scaling: Optional[dict]) -> torch.Tensor:
    """float32 [rot_dim / 2], computed in the reference's order of float32 operations."""
    inv = 1.0 / (theta ** (torch.arange(0, rot_dim, 2).float() / rot_dim))
    if not scaling:
        return inv
    kind = scaling.get("rope_type", "default")
    if kind == "default":
        return inv
    if kind != "llama3":
        raise ValueError(f"rotary scaling {kind!r} is not supported (default, llama3)")
    factor = float(scaling["factor"])
    low = float(scaling["low_freq_factor"])
    high = float(scaling["high_freq_factor"])
    orig = float(scaling["original_max_position_embeddings"])
    wavelen = 2 * math.pi / inv
    low_wavelen, high_wavelen = orig / low, orig / high
    scaled = torch.where(wavelen > low_wavelen, inv / factor, inv)
    smooth = (orig / wavelen - low) / (high - low)
    blended = (1 - smooth) * scaled / factor + smooth * scaled
    medium = (~(wavelen < high_wavelen)) & (~(wavelen > low_wavelen))
    return torch.where(medium, blended, scaled)


class RotaryEncoding(PositionEncoding):
    """params: rot_dim (how many leading elements of a head are rotated), theta, scaling
    (None or {"rope_type": "llama3", factor, low_freq_factor, high_freq_factor,
    original_max_position_embeddings})."""

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        self.rot_dim = int(params["rot_dim"])
        if self.rot_dim <= 0 or self.rot_dim % 2:
            raise ValueError(f"rot_dim must be positive and even, got {self.rot_dim}")
        self.theta = float(params["theta"])
        self.scaling = params.get("scaling")
        inv = inverse_frequencies(self.rot_dim, self.theta, self.scaling)
        self.inv_freq = inv
        pos = torch.arange(runtime.max_positions, dtype=torch.float32)
        angle = torch.outer(pos, inv).float()
        table = torch.stack([torch.cos(angle), torch.sin(angle)], dim=-1)       # [P, rot/2, 2]
        self.table = table.contiguous().to(runtime.device)

    def fused_table(self, head_dim: int):
        """The (cos, sin) table, if a product kernel may apply this encoding in its own epilogue:
        that needs the whole head to be rotated."""
        return self.table if self.rot_dim == head_dim else None

    def encode_and_store(self, qkv, ctx, kv, n_q, n_kv, head_dim, write_kv):
        q = torch.empty((qkv.shape[0], n_q * head_dim), dtype=qkv.dtype, device=qkv.device)
        ops.rope_store(qkv, q, kv.k if kv is not None else None, kv.v if kv is not None else None, self.table,
                       ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, kv.block_table, kv.page_size, n_q, n_kv, head_dim,
                       self.rot_dim, write_kv)
        return q


class NoEncoding(PositionEncoding):
    """Positions enter nowhere: keys and values are stored as projected."""

    def encode_and_store(self, qkv, ctx, kv, n_q, n_kv, head_dim, write_kv):
        q = torch.empty((qkv.shape[0], n_q * head_dim), dtype=qkv.dtype, device=qkv.device)
        ops.rope_store(qkv, q, kv.k, kv.v, None, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, kv.block_table,
                       kv.page_size, n_q, n_kv, head_dim, 0, write_kv)
        return q


register_position_encoding("rope", RotaryEncoding)
register_position_encoding("none", NoEncoding)
