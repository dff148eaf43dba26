"""Architecture-neutral description of a decoder: what the model builder consumes.

A typed, architecture-specific configuration (for instance `LlamaConfig`) is turned into a
`ModelSpec` by its architecture's `to_spec` function. From there on nothing knows the
architecture's name: parts are chosen layer by layer by `PartSpec.kind` through the part
registries, every size and constant is a parameter of the part, and the order in which
layers run is the `schedule` list.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Sequence


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: the registry key of its implementation and its parameters."""
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: how its parts are arranged (the block kind), the parts themselves, and the
    checkpoint sub-names under which each part's tensors are stored."""
    block: str                                   # registry key of the arrangement, e.g. "pre_norm"
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec
    names: Mapping[str, str]                     # part role -> checkpoint sub-name


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
