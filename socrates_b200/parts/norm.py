"""RMSNorm: y = x / sqrt(mean(x^2) + eps) * w, eps inside the root, gain w itself.

The reference computes it in the activations' dtype (model/qwen/qwen_kv_cont.py:45-53);
here the sum of squares, the root and the product are float32 and only the result is
rounded to the model dtype.  The kernel also adds the pending branch output to the
residual first, which is the residual sum of the block.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..kernels import ops
from .base import ParamSpec, Part, ResidualStream, register_part


class RMSNorm(Part):
    def __init__(self, spec, name):
        super().__init__(spec, name)
        self.dim = int(spec.params["dim"])
        self.eps = float(spec.params["eps"])
        self.gain: Optional[torch.Tensor] = None

    def parameters(self) -> Dict[str, ParamSpec]:
        return {self.name + "weight": ParamSpec((self.dim,), role="gain", init="gain")}

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype) -> None:
        self.gain = tensors[self.name + "weight"]

    def apply(self, ctx, stream: ResidualStream, row_index: Optional[torch.Tensor] = None,
              buffer: str = "normed") -> torch.Tensor:
        """Fold the pending branch into the residual and return the normed rows.

        With `row_index` only those rows are normed (for the head) and the residual
        is left unchanged.
        """
        M = stream.residual.shape[0] if row_index is None else row_index.numel()
        take = ctx.buffers.take if row_index is None else ctx.buffers.take_wanted
        out = take(buffer, M, (self.dim,), ctx.dtype)
        delta = stream.pending.partial if stream.pending is not None else None
        ops.add_rmsnorm(stream.residual, delta, self.gain, out, self.eps, row_index)
        if row_index is None:
            stream.pending = None
        return out


register_part("norm", "rmsnorm", RMSNorm)
