"""A model built from a plan: embedding, layers run in the plan's order, norm, head.

Nothing here names an architecture.  `Model(plan)` builds every part through the part
registries; `parameters()` lists the tensors the checkpoint must hold; `bind()` hands
them out; `forward(ctx, cache)` runs one step and returns float32 logits at the rows
named by `ctx.logit_index`.
"""

from __future__ import annotations

from typing import Dict, List, Mapping, Optional

import torch

from ..cache.manager import CacheNeeds
from ..config.plan import ModelPlan
from ..parts import ParamSpec, ResidualStream, build_part
from ..parts.base import _REGISTRIES
from .context import CacheView, StepContext


class Model:
    def __init__(self, plan: ModelPlan):
        plan.validate()
        self.plan = plan
        self.embedding = build_part("embedding", plan.embedding, plan.embedding.name)
        self.layers = []
        for spec in plan.layers:
            reg = _REGISTRIES["arrangement"]
            if spec.arrangement not in reg:
                raise KeyError(f"no arrangement {spec.arrangement!r}; known: {sorted(reg)}")
            self.layers.append(reg[spec.arrangement](spec))
        self.final_norm = build_part("norm", plan.final_norm, plan.final_norm.name)
        self.head = build_part("head", plan.head, plan.head.name)
        self.dtype: Optional[torch.dtype] = None

    # ------------------------------------------------------------------ weights
    def parameters(self) -> Dict[str, ParamSpec]:
        out: Dict[str, ParamSpec] = {}
        for part in (self.embedding, *self.layers, self.final_norm, self.head):
            for name, spec in part.parameters().items():
                if name in out and out[name].shape != spec.shape:
                    raise ValueError(f"{name} is asked for with shapes {out[name].shape} and {spec.shape}")
                out[name] = spec
        return out

    def duplicates(self) -> Dict[str, str]:
        """Tensors a checkpoint may hold beside the one a part reads ({file name: the name it must
        repeat}); parts say so through an optional `duplicates()`."""
        out: Dict[str, str] = {}
        for part in (self.embedding, *self.layers, self.final_norm, self.head):
            out.update(getattr(part, "duplicates", dict)())
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype) -> None:
        self.dtype = dtype
        for part in (self.embedding, *self.layers, self.final_norm, self.head):
            part.bind(tensors, dtype)
        # The weight matrices in the order in which a step streams them (parts that say so
        # through streamed_weights()), as a map from each one's address to its successor: a
        # kernel that streams one can ask for the head of the next in L2.
        order: List[torch.Tensor] = []
        for e in self.plan.order:
            order.extend(getattr(self.layers[e.layer], "streamed_weights", list)())
        order.extend(getattr(self.head, "streamed_weights", list)())
        self.weight_successor: Dict[int, torch.Tensor] = {}
        for w, nxt in zip(order, order[1:]):
            self.weight_successor.setdefault(w.data_ptr(), nxt)

    # ------------------------------------------------------------------ cache
    def cache_needs(self) -> List[Optional[CacheNeeds]]:
        """What each order entry asks of the cache manager (None where it reads another's)."""
        out: List[Optional[CacheNeeds]] = []
        for e in self.plan.order:
            out.append(None if e.reads_cache_of is not None else self.layers[e.layer].cache_needs())
        return out

    @property
    def supports_graph(self) -> bool:
        return all(l.supports_graph for l in self.layers)

    # ------------------------------------------------------------------ one step
    def forward(self, ctx: StepContext, cache) -> torch.Tensor:
        ctx.weight_successor = self.weight_successor
        stream = ResidualStream(self.embedding.forward(ctx))
        for i, e in enumerate(self.plan.order):
            src = e.reads_cache_of
            view = CacheView(cache, i if src is None else src, writes=src is None)
            self.layers[e.layer].forward(ctx, stream, view)
        if ctx.logit_index is None:
            return None          # no logits wanted: the last branch is never needed
        h = self.final_norm.apply(ctx, stream, row_index=ctx.logit_index, buffer="normed_out")
        return self.head.forward(ctx, h)
