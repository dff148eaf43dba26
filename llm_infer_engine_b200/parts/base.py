"""Interfaces and registries of the parts a layer is put together from.

Six kinds of part, each with a registry from a kind name to a class:

    mixer              x[T, d] -> [T, d], mixes information between positions; may own cache
    feed_forward       x[T, d] -> [T, d], position-wise
    norm               float32 residual rows -> normalised activations
    position_encoding  how positions enter a mixer (rotation of q and k here)
    pointwise          a float32 tensor -> the same tensor changed row by row; the model's two optional
                       slots outside the layers (after the embedding, after the head)
    block              the arrangement of a layer's parts around the residual stream; it declares the
                       roles it has (`ROLES`) and the part group of each

A part is constructed from `(params, runtime)`: `params` is the mapping of its `PartSpec`
(every size and constant it needs; nothing is read from a model-wide config), `runtime` says
where and in which precision it runs. It declares its checkpoint tensors with `param_specs()`
and receives them through `load()`. No part knows which model it is in.

Adding a part: subclass the interface, then `register_mixer("my_kind", MyMixer)` (or the
matching function); a `PartSpec("my_kind", {...})` in a `ModelSpec` now builds it.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Dict, List, Mapping, Optional, Tuple, Union

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


@dataclass(frozen=True)
class AttentionOptions:
    """Everything about softmax(q k^T) v that is not a shape. A mixer fills one and hands it to
    `ctx.attention`; a further option (a score cap, a bias by distance) becomes a field here with a
    default that means "off", and `KernelPlan.attention` sends a call that sets it to a kernel that
    knows it (the plain kernel first), so the call sites of the existing options do not change."""
    scale: float
    window: int = 0              # 0 = every earlier key; n = the last n keys, the token's own included


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
    """Two class flags widen what a block hands to `forward`; both default to False, and a part that
    leaves them so is called with exactly `(x, ctx, unit, owns_cache)`:

    accepts_deferred_norm  x may be a `DeferredNorm` instead of a tensor: the part folds the norm into
                           its first kernel, or calls `x.apply()` and goes on with the tensor.
    adds_to_residual       the block also passes `residual=h` (the float32 residual stream [T, d]); the
                           part may add its output into it inside its last kernel and then returns None
                           instead of a branch output, or ignores it and returns the output as usual.
    """
    accepts_deferred_norm = False
    adds_to_residual = False

    def cache_requests(self) -> List[object]:
        """KVRequest / StateRequest objects: what one run of this mixer needs per sequence."""
        return []

    def forward(self, x: Union[torch.Tensor, "DeferredNorm"], ctx, unit, owns_cache: bool,
                residual: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """x: normalised activations [T, d] (or a DeferredNorm, see the class flags). `unit` is the
        CacheUnit to use; when `owns_cache` is False it belongs to an earlier schedule entry and must
        only be read. Returns the branch output [T, d], or None after adding it into `residual`."""
        raise NotImplementedError


class FeedForward(Part):
    """The class flags of `Mixer` hold here too, with the call `(x, ctx)` as the plain form."""
    accepts_deferred_norm = False
    adds_to_residual = False

    def forward(self, x: Union[torch.Tensor, "DeferredNorm"], ctx,
                residual: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        raise NotImplementedError


class Pointwise(Part):
    """A change of a float32 tensor row by row, for the model's two slots outside the layers."""

    def forward(self, x: torch.Tensor, ctx, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x: float32 [n, width], changed in place or replaced by the returned tensor. After the embedding
        row i is token i of the step (`ctx.tok_pos[i]` is its position) and `rows` is None; after the head
        row i is the logits of packed token `rows[i]`."""
        raise NotImplementedError


def call_branch(part, x, ctx, *cache_args, residual: Optional[torch.Tensor] = None):
    """Calls a mixer or feed-forward the way its class flags ask for: `residual` is passed only to a part
    that declared `adds_to_residual`, and a DeferredNorm is applied first unless the part accepts one."""
    if isinstance(x, DeferredNorm) and not part.accepts_deferred_norm:
        x = x.apply()
    if part.adds_to_residual and residual is not None:
        return part.forward(x, ctx, *cache_args, residual=residual)
    return part.forward(x, ctx, *cache_args)


class Block:
    """Arrangement of one layer's parts around the float32 residual stream.

    A subclass declares `ROLES`: role name -> part group ("mixer", "feed_forward", "norm", ...). The model
    builder builds one part per role from the layer's `LayerSpec.parts` and hands them over as a dict;
    each is then an attribute of the block under its role name.

    forward(h, pending, ctx, unit, owns_cache) -> (h, pending): `pending` is a branch output
    not yet added to h (None at the first layer), so that each residual add can be fused with
    the norm that follows it."""
    ROLES: Dict[str, str] = {}

    def __init__(self, parts: Dict[str, Part], runtime: Runtime):
        missing = [r for r in self.ROLES if r not in parts]
        unknown = [r for r in parts if r not in self.ROLES]
        if missing or unknown:
            raise ValueError(f"{type(self).__name__} has the roles {sorted(self.ROLES)}; missing {missing}, "
                             f"unknown {unknown}")
        clash = [r for r in self.ROLES if hasattr(Block, r) or r in ("runtime", "_parts")]
        if clash:
            raise ValueError(f"{type(self).__name__}: role name(s) {clash} collide with the block's own attributes")
        self._parts = {role: parts[role] for role in self.ROLES}
        self.runtime = runtime
        for role, part in self._parts.items():
            setattr(self, role, part)

    def parts(self) -> Dict[str, Part]:
        return dict(self._parts)

    def mixer_roles(self) -> List[str]:
        return [role for role, group in self.ROLES.items() if group == "mixer"]

    def cache_requests(self) -> List[object]:
        """What one run of this layer needs per sequence: the requests of its mixers. With one mixer they
        are the mixer's own; with several, each request's name is prefixed with the mixer's role
        ("role.name") and `unit.scoped(role)` gives that mixer its own view."""
        roles = self.mixer_roles()
        if len(roles) == 1:
            return list(self._parts[roles[0]].cache_requests())
        out = []
        for role in roles:
            for r in self._parts[role].cache_requests():
                out.append(dataclasses.replace(r, name=f"{role}.{r.name}"))
        return out

    def forward(self, h, pending, ctx, unit, owns_cache):
        raise NotImplementedError


_REGISTRIES: Dict[str, Dict[str, type]] = {"mixer": {}, "feed_forward": {}, "norm": {}, "position_encoding": {},
                                           "pointwise": {}, "block": {}}


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


def register_pointwise(kind: str, cls: type) -> None:
    _register("pointwise", kind, cls)


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
