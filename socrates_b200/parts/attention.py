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

import os
from typing import Dict, Mapping, Optional

import torch

from ..cache.manager import CacheNeeds, PagedKVSpec
from ..kernels import ops
from .base import Branch, ParamSpec, Part, build_part, register_part
from .linear import Linear


def paged_partition() -> Optional[int]:
    """PAGED_PARTITION as in the reference (model/kernels/__init__.py:23-41): keys per partition of
    the split-key decode attention, 0 = one pass over all keys; None for "auto" or unset."""
    v = os.environ.get("PAGED_PARTITION", "auto").strip().lower()
    if v in ("", "auto"):
        return None
    n = int(v)
    if n < 0:
        raise ValueError(f"PAGED_PARTITION must be 'auto' or a non-negative integer, not {v!r}")
    return n


def decode_partitions(ctx, num_kv_heads: int, blocks_per_sm: int, keys_per_part: int) -> int:
    """Into how many key partitions the split-key decode kernel cuts each token's keys when
    PAGED_PARTITION is "auto": as many as keep every block resident at once (one wave, no tail),
    at most 16, never less than `keys_per_part` keys of the longest possible row in a partition.
    A function of the batch width and of limits only, so that a recorded graph stays valid."""
    most = max(1, -(-ctx.max_context // keys_per_part))
    blocks = max(1, num_kv_heads * ctx.num_tokens)
    return max(1, min((ctx.num_sms * blocks_per_sm) // blocks, most, 16))


def paged_attention(ctx, out, q, k_pool, v_pool, table, num_heads: int, scale: float, window: int,
                    max_len: int) -> None:
    """Causal attention of every token of the step over its row's pages; this mixer's choice of kernel.

    bfloat16, a step in which every request brings one token (decode):
      * PAGED_PARTITION "auto": the split-key kernel (mma.sync), the partition COUNT chosen from
        the batch width so that one wave of blocks fills the GPU.  Fastest; a request's numbers
        differ in rounding with the width of the batch it is in.
      * PAGED_PARTITION = n: the streaming kernel over chunks of n keys at fixed key positions (the
        reference's meaning of the variable, model/kernels/csrc/paged_attention.cu:80-96; 0 = the
        whole row in one pass).  A request's numbers are the same bits alone and in a full batch;
        measured 12 to 25 % slower per decode step than "auto" on the 4B shape.
    bfloat16, other steps: the tile kernels (tcgen05 for head sizes 64 and 128, mma.sync for 16 and
    32).  Everything else (the float32 engine above all): the SIMT kernel, whose split depends on
    `max_len` of the cache alone, so the float32 engine's numbers never depend on the batch.
    """
    Hkv, page_size, D = k_pool.shape[1], k_pool.shape[2], k_pool.shape[3]
    N = q.shape[0]
    bf16 = q.dtype == torch.bfloat16
    if bf16 and not ctx.all_decode:
        if ctx.status is not None and ops.attention_tcgen05_supports(num_heads, Hkv, D, page_size):
            ops.attention_prefill_tcgen05(out, q, k_pool, v_pool, table, ctx.seq_starts, ctx.seq_rows,
                                          ctx.seq_first_pos, num_heads, scale, ctx.status, window)
            return
        if ops.attention_mma_supports(num_heads, Hkv, D, page_size, False):
            ops.attention_prefill_mma(out, q, k_pool, v_pool, table, ctx.seq_starts, ctx.seq_rows,
                                      ctx.seq_first_pos, num_heads, scale, window)
            return
    fixed = paged_partition()
    take = ctx.buffers.take_flat
    if (bf16 and ctx.all_decode and fixed is not None and N <= 1024      # the kernel's limit of tokens a launch
            and ops.attention_decode_stream_supports(num_heads, Hkv, D, page_size)):
        chunk = max(16, -(-(fixed if fixed > 0 else max_len) // 16) * 16)
        span = min(max_len, window) if window else max_len
        chunks = 1 if chunk >= max_len else -(-span // chunk) + 1          # a span may straddle one edge more
        part_o = part_ml = counters = None
        if chunks > 1:
            part_o = take("attn_part_o", N * num_heads * chunks * D, torch.float32)
            part_ml = take("attn_part_ml", N * num_heads * chunks * 2, torch.float32)
            counters = take("attn_counters", ctx.buffers.max_rows * Hkv, torch.int32, zeroed=True)
        ops.attention_decode_stream(out, q, k_pool, v_pool, table, ctx.token_rows, ctx.positions, num_heads,
                                    scale, window, chunk, chunks, part_o, part_ml, counters,
                                    variant=int(os.environ.get("SOCRATES_DECODE_VARIANT", "1")))
        return
    use_mma = bf16 and ctx.all_decode and ops.attention_mma_supports(num_heads, Hkv, D, page_size, True)
    if use_mma:
        NP = decode_partitions(ctx, Hkv, ops.attention_decode_mma_blocks_per_sm(D), 128)
    else:
        # SIMT: a partition is ceil(pages of the row / NP) pages, so a fixed NP cuts a row by its own length alone
        keys_per_part = 4 * page_size if fixed is None else fixed
        NP = 1 if keys_per_part == 0 else max(1, min(-(-max_len // keys_per_part), 16))
    part_o = part_ml = None
    if NP > 1:
        part_o = take("attn_part_o", N * num_heads * NP * D, torch.float32)
        part_ml = take("attn_part_ml", N * num_heads * NP * 2, torch.float32)
    if use_mma:
        ops.attention_decode_mma(out, q, k_pool, v_pool, table, ctx.token_rows, ctx.positions, num_heads,
                                 scale, window, NP, part_o, part_ml)
    else:
        ops.attention_simt(out, q, k_pool, v_pool, table, ctx.token_rows, ctx.positions, num_heads, scale,
                           window, NP, part_o, part_ml)


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
        paged_attention(ctx, attn, q, k_pool, v_pool, table, self.Hq, self.scale, self.window or 0,
                        cache.manager.max_len)
        return Branch(self.o(ctx, attn, "branch", out="partial"))


register_part("mixer", "gqa_attention", GQAAttention)
