"""Interfaces and registries of the parts a layer is put together from.

Five kinds of part, each with a registry from a kind name to a class:

    mixer              x[T, d] -> [T, d], mixes information between positions; may own cache
    feed_forward       x[T, d] -> [T, d], position-wise
    norm               float32 residual rows -> normalised activations
    position_encoding  how positions enter a mixer (rotation of q and k here)
    block              the arrangement of mixer, feed-forward and norms around the residual stream

A part is constructed from `(params, runtime)`: `params` is the mapping of its `PartSpec`
(every size and constant it needs; nothing is read from a model-wide config), `runtime` says
where and in which precision it runs. It declares its checkpoint tensors with `param_specs()`
and receives them through `load()`. No part knows which model it is in.

Adding a part: subclass the interface, then `register_mixer("my_kind", MyMixer)` (or the
matching function); a `PartSpec("my_kind", {...})` in a `ModelSpec` now builds it.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Mapping, Optional, Tuple

import torch


@dataclass(frozen=True)
class Runtime:
    device: torch.device
    dtype: torch.dtype            # activation dtype: torch.float32 (true 32-bit path) or torch.bfloat16
    max_positions: int            # longest sequence the engine will hold


@dataclass(frozen=True)
class ParamSpec:
    """A checkpoint tensor of a part. `role`: "matrix" (a GEMM operand), "vector" (norm weights,
    biases) or "table" (integers). `init` is how the random-weights mode fills it:
    ("normal",) uses the caller's std, ("ones",), ("zeros",) or ("uniform", lo, hi)."""
    shape: Tuple[int, ...]
    role: str = "matrix"
    init: Tuple = ("normal",)


class Part:
    def __init__(self, params: Mapping, runtime: Runtime):
        self.params = dict(params)
        self.runtime = runtime

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Receives the tensors named by param_specs(), already on the device."""

    def weight_bytes(self) -> int:
        """Bytes of weights that one step reads (for roofline accounting)."""
        return 0

    def stack_view(self) -> Optional[dict]:
        """What a kernel that runs a whole stack of layers by itself needs of this part: a dict with
        "kind" and the part's tensors and constants, or None when the part can only be run through
        forward(). The engine uses such a kernel only when every part of every layer gives a view
        that the kernel knows; anything else runs part by part."""
        return None


class Norm(Part):
    def forward(self, h: torch.Tensor, delta: Optional[torch.Tensor], out: Optional[torch.Tensor] = None,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """h (float32 [T, d]) += delta in place when rows is None; returns norm(h) in the
        activation dtype. With `rows`, only those rows are produced and h is untouched."""
        raise NotImplementedError

    def defer(self, h: torch.Tensor) -> Optional["DeferredNorm"]:
        """A promise of norm(h) for a consumer that can fold the norm into its own first kernel,
        or None when this norm (or this shape) cannot be folded."""
        return None


class DeferredNorm:
    """norm(h) that has not been computed. A part that declares `accepts_deferred_norm = True`
    may receive one instead of a tensor; it either folds the norm into its first kernel (using
    `kind`, `weight`, `eps`) or calls `apply()` and goes on with the tensor."""

    def __init__(self, norm: Norm, h: torch.Tensor, kind: str, weight: torch.Tensor, eps: float):
        self.norm, self.h, self.kind, self.weight, self.eps = norm, h, kind, weight, eps

    @property
    def shape(self):
        return self.h.shape

    def apply(self) -> torch.Tensor:
        return self.norm.forward(self.h, None)


class PositionEncoding(Part):
    def encode_and_store(self, qkv: torch.Tensor, ctx, kv, n_q: int, n_kv: int, head_dim: int,
                         write_kv: bool) -> torch.Tensor:
        """Takes the packed projections [T, (n_q + 2 n_kv) head_dim], returns position-encoded
        queries [T, n_q head_dim] and, if write_kv, writes encoded keys and the values into
        the cache unit `kv` at each token's position."""
        raise NotImplementedError


class Mixer(Part):
    def cache_requests(self) -> List[object]:
        """KVRequest / StateRequest objects: what one run of this mixer needs per sequence."""
        return []

    def forward(self, x: torch.Tensor, ctx, unit, owns_cache: bool) -> torch.Tensor:
        """x: normalised activations [T, d]. `unit` is the CacheUnit to use; when `owns_cache`
        is False it belongs to an earlier schedule entry and must only be read."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError


class Block:
    """Arrangement of one layer's parts around the float32 residual stream.

    forward(h, pending, ctx, unit, owns_cache) -> (h, pending): `pending` is a branch output
    not yet added to h (None at the first layer), so that each residual add can be fused with
    the norm that follows it."""

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm, feed_forward_norm: Norm,
                 runtime: Runtime):
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.feed_forward_norm = feed_forward_norm
        self.runtime = runtime

    def parts(self) -> Dict[str, Part]:
        return {"mixer": self.mixer, "feed_forward": self.feed_forward, "mixer_norm": self.mixer_norm,
                "feed_forward_norm": self.feed_forward_norm}

    def forward(self, h, pending, ctx, unit, owns_cache):
        raise NotImplementedError

    def stack_view(self) -> Optional[dict]:
        """As Part.stack_view, for the arrangement: "kind" plus the views of the four parts."""
        return None


_REGISTRIES: Dict[str, Dict[str, type]] = {"mixer": {}, "feed_forward": {}, "norm": {}, "position_encoding": {},
                                           "block": {}}


def _register(group: str, kind: str, cls: type) -> None:
    _REGISTRIES[group][kind] = cls


def register_mixer(kind: str, cls: type) -> None:
    _register("mixer", kind, cls)


def register_feed_forward(kind: str, cls: type) -> None:
    _register("feed_forward", kind, cls)


def register_norm(kind: str, cls: type) -> None:
    _register("norm", kind, cls)


def register_position_encoding(kind: str, cls: type) -> None:
    _register("position_encoding", kind, cls)


def register_block(kind: str, cls: type) -> None:
    _register("block", kind, cls)


def lookup(group: str, kind: str) -> type:
    reg = _REGISTRIES[group]
    if kind not in reg:
        raise KeyError(f"no {group} of kind {kind!r} is registered (known: {sorted(reg)})")
    return reg[kind]


def undefer(x):
    """The tensor behind x, applying a deferred norm if x is one."""
    return x.apply() if isinstance(x, DeferredNorm) else x


def build_part(group: str, spec, runtime: Runtime):
    """spec: a PartSpec (or anything with .kind and .params)."""
    return lookup(group, spec.kind)(spec.params, runtime)
