"""y = x W^T for a weight matrix [out, in] (torch.nn.Linear layout, no bias).

`Linear` chooses the kernel: the float32 path and shapes the tensor-core kernel does
not take run on the CUDA cores (`gemm_simt`); bfloat16 runs on the tcgen05 kernel when
it is loaded.  The output is the model dtype `[M, N]`, float32 `[M, N]` (logits), or
float32 partial sums `[S, M, N]` for a branch that the next norm adds to the residual.
"""

from __future__ import annotations

import torch

from ..kernels import ops


class Linear:
    def __init__(self, weight: torch.Tensor):
        if weight.dim() != 2:
            raise ValueError(f"a weight matrix has two dims, got {tuple(weight.shape)}")
        self.weight = weight.contiguous()
        self.out_features, self.in_features = weight.shape

    def __call__(self, ctx, x: torch.Tensor, buffer: str, out: str = "model", epilogue: int = 0) -> torch.Tensor:
        """`out`: "model" -> [M, N] in the model dtype; "float32" -> [M, N] float32;
        "wanted_float32" -> the same for rows that are wanted logits (a buffer of its own size);
        "partial" -> float32 [S, M, N]; "model_or_partial" -> partial sums when the
        product is cut along K (the weight-streaming regime), else the model dtype: for
        consumers that can add the parts themselves."""
        M = x.shape[0]
        N = self.out_features // 2 if epilogue == 1 else self.out_features
        if out == "model_or_partial":
            out = "partial" if ctx.gemm_splits(M, self.weight, x.dtype, shares=False) > 1 else "model"
        if out == "model":
            y = ctx.buffers.take(buffer, M, (N,), ctx.dtype)
        elif out == "float32":
            y = ctx.buffers.take(buffer, M, (N,), torch.float32)
        elif out == "wanted_float32":
            y = ctx.buffers.take_wanted(buffer, M, (N,), torch.float32)
        elif out == "partial":
            S = ctx.gemm_splits(M, self.weight, x.dtype)
            y = ctx.buffers.take_flat(buffer, S * M * N, torch.float32).view(S, M, N)
        else:
            raise ValueError(out)
        ctx.gemm(y, x, self.weight, epilogue)
        return y
