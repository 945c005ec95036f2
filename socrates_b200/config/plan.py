"""Data that describes a model: parts by kind, layers, and the order they run in.

A model is not a class hierarchy here. An architecture's configuration produces a
`ModelPlan`; the generic model builder turns every `PartSpec` in it into a part
object through the registries in `socrates_b200.parts`. Nothing in a plan knows
which architecture produced it, and no part knows which plan it sits in.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part: a registered `kind` and the sizes and constants it is built with."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    # Checkpoint name prefix of this part's tensors, relative to its parent
    # (the layer prefix for parts of a layer, nothing for parts of the model).
    name: str = ""

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    """One layer's weights and parts.

    `arrangement` names how the parts are wired (registered in
    `socrates_b200.parts.block`); `prefix` is the checkpoint name prefix of the
    layer's tensors, e.g. ``model.layers.3.``.
    """

    arrangement: str
    prefix: str
    norms: Tuple[PartSpec, ...]
    mixer: PartSpec
    feed_forward: PartSpec


@dataclass(frozen=True)
class RunEntry:
    """One execution of a layer.

    `layer` indexes `ModelPlan.layers` and may repeat: the same weights run twice,
    each run with a cache of its own.  `reads_cache_of` names an earlier entry (by
    its index in `ModelPlan.order`) whose cache this run reads instead of writing
    one of its own.
    """

    layer: int
    reads_cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelPlan:
    architecture: str
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    order: Tuple[RunEntry, ...]
    final_norm: PartSpec
    head: PartSpec

    def validate(self) -> None:
        for i, e in enumerate(self.order):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"order[{i}] names layer {e.layer}; the plan has {len(self.layers)}")
            if e.reads_cache_of is not None:
                if not 0 <= e.reads_cache_of < i:
                    raise ValueError(
                        f"order[{i}] reads the cache of entry {e.reads_cache_of}, "
                        f"which does not run before it")
                if self.order[e.reads_cache_of].reads_cache_of is not None:
                    raise ValueError(
                        f"order[{i}] reads the cache of entry {e.reads_cache_of}, "
                        f"which has no cache of its own")
