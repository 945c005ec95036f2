"""Interfaces of the parts a model is put together from, and their registries.

A part is built from a `PartSpec` (its sizes and constants), declares the tensors it
needs by name, receives them once (`bind`), and then runs on the tokens of a step.
No part knows which model it sits in; which part a layer uses is decided layer by
layer by the plan.  The five kinds and what each must provide:

* **norm**           `apply(ctx, stream, row_index=None) -> normed [M, d]`: folds the
                     stream's pending branch output into the residual and norms it.
* **position**       `tables() -> (inv_freq float32 [rotary_dim/2], rotary_dim)`:
                     what the mixer's rotation kernel multiplies positions with.
* **mixer**          `cache_needs() -> CacheNeeds | None` and
                     `forward(ctx, x [N, d], cache: CacheView) -> Branch`.
* **feed_forward**   `forward(ctx, x [N, d]) -> Branch`.
* **arrangement**    `forward(ctx, stream, cache: CacheView)`: wires norms, mixer and
                     feed-forward of one layer around the residual stream.

A `Branch` is the float32 output of a mixer or feed-forward as `S` partial sums
`[S, N, d]` (S > 1 when the last matrix product was split along K); the next norm
adds them to the residual in a fixed order, so the sum costs no pass of its own.

To add a part: subclass `Part`, give it `parameters()`, `bind()` and the method of
its kind, and call `register_part(kind_group, name, cls)`.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Mapping, Optional, Tuple

import torch

from ..config.plan import PartSpec


@dataclass(frozen=True)
class ParamSpec:
    """One tensor a part expects: its shape, and how random weights are drawn for it.

    role "matrix": a weight matrix, kept in the model dtype (bfloat16 or float32).
    role "gain":   a norm gain, always held as float32 on the device.
    init "normal": N(0, 0.02); init "gain": 1 + N(0, 0.1).
    """
    shape: Tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"


class Part:
    """Base of all parts.  `name` is the full checkpoint prefix of the part's tensors."""

    def __init__(self, spec: PartSpec, name: str):
        self.spec = spec
        self.name = name

    def parameters(self) -> Dict[str, ParamSpec]:
        """Full checkpoint name -> ParamSpec of every tensor this part reads."""
        return {}

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype) -> None:
        """Receive the tensors named by `parameters()`, already on the device."""

    supports_graph = True   # False if forward() needs host values that change per step


@dataclass
class Branch:
    """Float32 partial sums `[S, N, d]` waiting to be added to the residual."""
    partial: torch.Tensor


class ResidualStream:
    """The float32 residual `[N, d]` of a step and the branch output not yet added."""

    def __init__(self, residual: torch.Tensor):
        self.residual = residual
        self.pending: Optional[Branch] = None


_REGISTRIES: Dict[str, Dict[str, Callable]] = {
    "norm": {}, "position": {}, "mixer": {}, "feed_forward": {}, "arrangement": {},
    "embedding": {}, "head": {},
}


def register_part(group: str, kind: str, factory: Callable, *, replace: bool = False) -> None:
    """Make `factory(spec, name)` (or, for arrangements, `factory(layer_spec, parts...)`)
    available under `kind` in one of the groups above."""
    if group not in _REGISTRIES:
        raise KeyError(f"unknown part group {group!r}; known: {sorted(_REGISTRIES)}")
    if kind in _REGISTRIES[group] and not replace:
        raise ValueError(f"{group} kind {kind!r} is already registered")
    _REGISTRIES[group][kind] = factory


def unregister_part(group: str, kind: str) -> None:
    _REGISTRIES[group].pop(kind, None)


def build_part(group: str, spec: PartSpec, name: str):
    reg = _REGISTRIES[group]
    if spec.kind not in reg:
        raise KeyError(f"no {group} of kind {spec.kind!r}; known: {sorted(reg)}")
    return reg[spec.kind](spec, name)


def registered(group: str) -> list[str]:
    return sorted(_REGISTRIES[group])
