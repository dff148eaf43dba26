"""Architecture-neutral description of a decoder: what the model builder consumes.

A typed, architecture-specific configuration (for instance `LlamaConfig`) is turned into a
`ModelSpec` by its architecture's `to_spec` function. From there on nothing knows the
architecture's name: parts are chosen layer by layer by `PartSpec.kind` through the part
registries, every size and constant is a parameter of the part, and the order in which
layers run is the `schedule` list.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from types import MappingProxyType
from typing import Any, Mapping, Optional, Sequence


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: the registry key of its implementation and its parameters."""
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


class LayerSpec:
    """One layer: how its parts are arranged (the block kind), the parts themselves by ROLE, and the
    checkpoint sub-names under which each role's tensors are stored.

    Which roles a layer has is the block's business: every `Block` subclass declares its roles and the
    part group of each (`Block.ROLES`), and the model builder checks the layer against it. The classic
    pre-norm block has four (`mixer`, `feed_forward`, `mixer_norm`, `feed_forward_norm`), and for it
    the short forms below exist; a block with three norms, a second mixer or one shared norm simply
    names other roles in `parts`.

        LayerSpec("pre_norm", mixer, feed_forward, mixer_norm, feed_forward_norm, names)
        LayerSpec(block="pre_norm", mixer=..., feed_forward=..., mixer_norm=..., feed_forward_norm=..., names=...)
        LayerSpec("my_block", parts={"mixer": ..., "mixer_norm": ..., "post_norm": ..., ...}, names={...})

    A role can be read as an attribute (`layer.mixer`)."""
    CLASSIC_ROLES = ("mixer", "feed_forward", "mixer_norm", "feed_forward_norm")

    def __init__(self, block: str, *classic, parts: Optional[Mapping[str, PartSpec]] = None,
                 names: Optional[Mapping[str, str]] = None, **by_role: PartSpec):
        if len(classic) > 5:
            raise TypeError("LayerSpec takes at most four positional parts and the names")
        if len(classic) == 5:
            if names is not None:
                raise TypeError("LayerSpec: names given twice")
            names = classic[4]
        roles = dict(parts or {})
        for role, spec in list(zip(self.CLASSIC_ROLES, classic[:4])) + list(by_role.items()):
            if role in roles:
                raise TypeError(f"LayerSpec: role {role!r} given twice")
            roles[role] = spec
        for role, spec in roles.items():
            if not hasattr(spec, "kind") or not hasattr(spec, "params"):
                raise TypeError(f"LayerSpec: role {role!r} must be a PartSpec, got {type(spec).__name__}")
        names = dict(names or {})
        unnamed = [r for r in roles if r not in names]
        if unnamed:
            raise ValueError(f"LayerSpec: no checkpoint sub-name for role(s) {unnamed}")
        object.__setattr__(self, "block", block)
        object.__setattr__(self, "parts", MappingProxyType(roles))
        object.__setattr__(self, "names", MappingProxyType(names))

    def __getattr__(self, role: str) -> PartSpec:
        parts = self.__dict__.get("parts")
        if parts is not None and role in parts:
            return parts[role]
        raise AttributeError(f"this layer ({self.__dict__.get('block')!r}) has no role {role!r}")

    def __setattr__(self, key, value):
        raise AttributeError("LayerSpec is read-only")

    def __repr__(self):
        return f"LayerSpec(block={self.block!r}, parts={dict(self.parts)!r}, names={dict(self.names)!r})"


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order. `layer` indexes `ModelSpec.layers`; a layer may appear in
    several entries. Each entry owns a cache unit of its own unless `cache_of` names an
    EARLIER entry of the schedule, whose unit it then reads instead of writing one."""
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    max_position: int
    layers: Sequence[LayerSpec]
    schedule: Sequence[LayerCall]
    final_norm: PartSpec
    tie_head: bool
    embedding_name: str                          # checkpoint name of the embedding table
    layer_prefix: str                            # e.g. "model.layers.{i}."
    final_norm_name: str
    head_name: str
    stop_token_ids: Sequence[int] = ()
    ignore_unexpected: Sequence[str] = ()        # regexes of checkpoint tensors to ignore
    # Two optional pointwise parts (group "pointwise") outside the layers: one on the float32 residual
    # stream right after the embedding gather (a scale, absolute position embeddings), one on the float32
    # logits of the wanted rows (a scale, a cap). Their tensors, if any, live under the given names.
    after_embedding: Optional[PartSpec] = None
    after_head: Optional[PartSpec] = None
    after_embedding_name: str = "after_embedding"
    after_head_name: str = "after_head"

    def validate(self) -> None:
        n = len(self.layers)
        for pos, call in enumerate(self.schedule):
            if not 0 <= call.layer < n:
                raise ValueError(f"schedule[{pos}] names layer {call.layer}, but there are {n} layers")
            if call.cache_of is not None:
                if not 0 <= call.cache_of < pos:
                    raise ValueError(
                        f"schedule[{pos}].cache_of = {call.cache_of} must name an earlier schedule entry")
                if self.schedule[call.cache_of].cache_of is not None:
                    raise ValueError(
                        f"schedule[{pos}].cache_of = {call.cache_of} names an entry that itself borrows a cache")
