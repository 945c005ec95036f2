"""SwiGLU feed-forward: down(up(x) * silu(gate(x))), no bias
(model/qwen/qwen_kv_cont.py:250-266).  gate and up are one matrix product here: when the
weights are bound their rows are interleaved (row 2f = gate_f, row 2f+1 = up_f), so that a
gate and its up value are neighbours in the product's output.  For many rows the
tensor-core kernel then applies SiLU*mul in its epilogue and the [N, 2F] intermediate is
never written; otherwise a SiLU*mul kernel reads the interleaved product.
silu(z) = z * sigmoid(z) in float32."""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..kernels import ops
from .base import Branch, ParamSpec, Part, register_part
from .linear import Linear


class SwiGLU(Part):
    def __init__(self, spec, name):
        super().__init__(spec, name)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.gate_up: Optional[Linear] = None
        self.down: Optional[Linear] = None

    def parameters(self) -> Dict[str, ParamSpec]:
        n = self.name
        return {
            n + "gate_proj.weight": ParamSpec((self.inter, self.hidden)),
            n + "up_proj.weight": ParamSpec((self.inter, self.hidden)),
            n + "down_proj.weight": ParamSpec((self.hidden, self.inter)),
        }

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype) -> None:
        n = self.name
        gate, up = tensors[n + "gate_proj.weight"], tensors[n + "up_proj.weight"]
        self.gate_up = Linear(torch.stack([gate, up], dim=1).reshape(2 * self.inter, self.hidden))
        self.down = Linear(tensors[n + "down_proj.weight"])

    def streamed_weights(self):
        """The weight matrices in the order in which forward() reads them."""
        return [self.gate_up.weight, self.down.weight]

    def forward(self, ctx, x: torch.Tensor) -> Branch:
        N = x.shape[0]
        if ctx.can_fuse_silu_mul(N, self.gate_up.weight, x.dtype):
            act = self.gate_up(ctx, x, "act", epilogue=1)
        else:
            gu = self.gate_up(ctx, x, "gate_up")
            act = ctx.buffers.take("act", N, (self.inter,), ctx.dtype)
            ops.silu_mul(act, gu, interleaved=True)
        return Branch(self.down(ctx, act, "branch", out="partial"))


register_part("feed_forward", "swiglu", SwiGLU)
