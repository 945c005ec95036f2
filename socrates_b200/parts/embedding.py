"""Token embedding and the output head.

Embedding: x = table[ids] (model/qwen/qwen_kv_paged.py:198,219), widened to the
float32 residual.  Head: logits = x W^T with W the embedding table when the
configuration ties them (:224) or `lm_head.weight` otherwise; only the rows whose
logits were asked for are computed, in float32.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..kernels import ops
from .base import ParamSpec, Part, register_part
from .linear import Linear


class Embedding(Part):
    def __init__(self, spec, name):
        super().__init__(spec, name)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.table: Optional[torch.Tensor] = None

    def parameters(self) -> Dict[str, ParamSpec]:
        return {self.name + "weight": ParamSpec((self.vocab, self.hidden))}

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype) -> None:
        self.table = tensors[self.name + "weight"]

    def forward(self, ctx) -> torch.Tensor:
        out = ctx.buffers.take("residual", ctx.num_tokens, (self.hidden,), torch.float32)
        ops.embed(out, self.table, ctx.token_ids, ctx.token_feedback)
        return out


class LMHead(Part):
    def __init__(self, spec, name):
        super().__init__(spec, name)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.tied_to: Optional[str] = spec.params.get("tied_to")
        self.linear: Optional[Linear] = None

    def parameters(self) -> Dict[str, ParamSpec]:
        if self.tied_to is not None:
            return {self.tied_to: ParamSpec((self.vocab, self.hidden))}
        return {self.name + "weight": ParamSpec((self.vocab, self.hidden))}

    def duplicates(self) -> Dict[str, str]:
        """A tied head reads the embedding; a file may still carry a copy under the head's name."""
        return {self.name + "weight": self.tied_to} if self.tied_to is not None else {}

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype) -> None:
        self.linear = Linear(tensors[self.tied_to or self.name + "weight"])

    def streamed_weights(self):
        return [self.linear.weight]

    def forward(self, ctx, x: torch.Tensor) -> torch.Tensor:
        return self.linear(ctx, x, "logits", out="wanted_float32")


register_part("embedding", "embedding", Embedding)
register_part("head", "lm_head", LMHead)
