"""How the parts of one layer are wired around the residual stream.

"pre_norm" is the reference's block (model/qwen/qwen_kv_paged.py:186-189):
x = x + mixer(norm_0(x)); x = x + feed_forward(norm_1(x)).  The additions happen
inside the next norm's kernel: each branch leaves its output pending on the stream
and the following norm (of this layer, the next layer, or the final one) folds it in.
"""

from __future__ import annotations

from typing import Dict, Mapping

from .base import ParamSpec, ResidualStream, build_part, register_part


class PreNormBlock:
    def __init__(self, layer_spec):
        if len(layer_spec.norms) != 2:
            raise ValueError("a pre_norm block has two norms")
        pre = layer_spec.prefix
        self.norms = [build_part("norm", s, pre + s.name) for s in layer_spec.norms]
        self.mixer = build_part("mixer", layer_spec.mixer, pre + layer_spec.mixer.name)
        self.feed_forward = build_part("feed_forward", layer_spec.feed_forward,
                                       pre + layer_spec.feed_forward.name)

    def parts(self):
        return [*self.norms, self.mixer, self.feed_forward]

    def parameters(self) -> Dict[str, ParamSpec]:
        out: Dict[str, ParamSpec] = {}
        for p in self.parts():
            out.update(p.parameters())
        return out

    def bind(self, tensors: Mapping, dtype) -> None:
        for p in self.parts():
            p.bind(tensors, dtype)

    @property
    def supports_graph(self) -> bool:
        return all(getattr(p, "supports_graph", True) for p in self.parts())

    def cache_needs(self):
        fn = getattr(self.mixer, "cache_needs", None)
        return fn() if fn is not None else None

    def streamed_weights(self):
        """Weight matrices in the order in which forward() streams them (optional for a part)."""
        return [*getattr(self.mixer, "streamed_weights", list)(),
                *getattr(self.feed_forward, "streamed_weights", list)()]

    def forward(self, ctx, stream: ResidualStream, cache) -> None:
        h = self.norms[0].apply(ctx, stream)
        stream.pending = self.mixer.forward(ctx, h, cache)
        h = self.norms[1].apply(ctx, stream)
        stream.pending = self.feed_forward.forward(ctx, h)


register_part("arrangement", "pre_norm", lambda layer_spec, name="": PreNormBlock(layer_spec))
