"""Grouped-query attention over the paged cache, with per-head QK-RMSNorm and rotation.

Formulas in the reference's order (model/qwen/qwen_kv_paged.py:130-175):
q, k, v = x Wq^T, x Wk^T, x Wv^T, viewed as heads of head_dim; q and k are RMS-normed
over head_dim with gains shared by all heads, then rotated by position; k and v go to
the row's pages; query head h attends over KV head h // G with scale head_dim^-0.5,
causally, optionally only over the last `window` keys; heads are concatenated and
projected by Wo.  The three projections are one matrix product here (the weights are
concatenated when they are bound).

Unlike the reference, whose prompt attention only sees the keys of the same call
(:166-174), every query reads its keys from the pages, so a prompt may arrive in
portions and portions of prompts share a step with decode tokens.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..cache.manager import CacheNeeds, PagedKVSpec
from ..kernels import ops
from .base import Branch, ParamSpec, Part, build_part, register_part
from .linear import Linear


class GQAAttention(Part):
    def __init__(self, spec, name):
        super().__init__(spec, name)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.Hq = int(p["num_heads"])
        self.Hkv = int(p["num_kv_heads"])
        self.D = int(p["head_dim"])
        self.scale = float(p.get("scale", self.D ** -0.5))
        self.qk_norm_eps = p.get("qk_norm_eps")          # None: no QK-norm
        self.window: Optional[int] = p.get("window")
        self.position = build_part("position", p["position"], "")
        if self.Hq % self.Hkv:
            raise ValueError(f"{self.Hq} query heads are no multiple of {self.Hkv} KV heads")
        if self.D % 16 or not 16 <= self.D <= 256:
            raise ValueError(f"head_dim {self.D} must be a multiple of 16 between 16 and 256")
        self.qkv: Optional[Linear] = None
        self.o: Optional[Linear] = None
        self.q_gain = self.k_gain = None

    def parameters(self) -> Dict[str, ParamSpec]:
        n, D = self.name, self.D
        out = {
            n + "q_proj.weight": ParamSpec((self.Hq * D, self.hidden)),
            n + "k_proj.weight": ParamSpec((self.Hkv * D, self.hidden)),
            n + "v_proj.weight": ParamSpec((self.Hkv * D, self.hidden)),
            n + "o_proj.weight": ParamSpec((self.hidden, self.Hq * D)),
        }
        if self.qk_norm_eps is not None:
            out[n + "q_norm.weight"] = ParamSpec((D,), role="gain", init="gain")
            out[n + "k_norm.weight"] = ParamSpec((D,), role="gain", init="gain")
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype) -> None:
        n = self.name
        self.qkv = Linear(torch.cat([tensors[n + "q_proj.weight"], tensors[n + "k_proj.weight"],
                                     tensors[n + "v_proj.weight"]], dim=0))
        self.o = Linear(tensors[n + "o_proj.weight"])
        if self.qk_norm_eps is not None:
            self.q_gain = tensors[n + "q_norm.weight"]
            self.k_gain = tensors[n + "k_norm.weight"]

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(paged=PagedKVSpec(self.Hkv, self.D, self.window))

    def streamed_weights(self):
        """The weight matrices in the order in which forward() reads them."""
        return [self.qkv.weight, self.o.weight]

    def forward(self, ctx, x: torch.Tensor, cache) -> Branch:
        N = x.shape[0]
        qkv = self.qkv(ctx, x, "qkv", out="model_or_partial")
        q = ctx.buffers.take("q", N, (self.Hq * self.D,), ctx.dtype)
        k_pool, v_pool = cache.pools()
        table = cache.block_table()
        inv_freq, rotary_dim = self.position.tables(x.device)
        eps = self.qk_norm_eps if self.qk_norm_eps is not None else 0.0
        ops.qk_norm_rope_kvwrite(
            qkv, q, k_pool if cache.writes else None, v_pool if cache.writes else None,
            self.q_gain, self.k_gain, inv_freq, rotary_dim, ctx.positions, ctx.token_rows, table,
            eps, self.Hq, self.Hkv, self.D)
        attn = ctx.buffers.take("attn", N, (self.Hq * self.D,), ctx.dtype)
        ctx.attention(attn, q, k_pool, v_pool, table, self.Hq, self.scale, self.window or 0)
        return Branch(self.o(ctx, attn, "branch", out="partial"))


register_part("mixer", "gqa_attention", GQAAttention)
