"""What a part sees of the step it runs in: the tokens, where they sit, and scratch.

A step is a flat batch of N tokens from R requests.  For token n the context gives
its id, its absolute position and the cache row of its request; for request r (in
batch order) the offset of its first token (`seq_starts`, R+1 entries), its cache row
and the position of its first token.  All of these are int32 device tensors that were
filled by one host-to-device copy before the step; no part reads anything back.
"""

from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..kernels import ops


class Buffers:
    """Scratch tensors of the step, by name, with addresses that never change.

    `take(name, rows, shape, dtype)` returns the first `rows` rows of a buffer that is
    allocated once for `max_rows` rows, so a CUDA graph that recorded its address stays
    valid.  `take_flat` serves buffers whose size does not scale with the row count; if
    one has to grow, the old storage is kept alive for the graphs that recorded it.
    """

    def __init__(self, max_rows: int, device):
        self.max_rows = max_rows
        self.device = device
        self._by_name: Dict[Tuple[str, tuple, torch.dtype], torch.Tensor] = {}
        self._flat: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}
        self._retired: List[torch.Tensor] = []

    def take(self, name: str, rows: int, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        if rows > self.max_rows:
            raise ValueError(f"{rows} rows exceed the step limit of {self.max_rows}")
        key = (name, tuple(shape), dtype)
        buf = self._by_name.get(key)
        if buf is None:
            buf = torch.empty((self.max_rows, *shape), dtype=dtype, device=self.device)
            self._by_name[key] = buf
        return buf[:rows]

    def take_flat(self, name: str, numel: int, dtype: torch.dtype) -> torch.Tensor:
        key = (name, dtype)
        buf = self._flat.get(key)
        if buf is None or buf.numel() < numel:
            if buf is not None:
                self._retired.append(buf)
            size = max(numel, 2 * buf.numel() if buf is not None else numel)
            buf = torch.empty(size, dtype=dtype, device=self.device)
            self._flat[key] = buf
        return buf[:numel]

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size()
                   for t in [*self._by_name.values(), *self._flat.values(), *self._retired])


class CacheView:
    """The cache as one run of one layer sees it."""

    def __init__(self, manager, entry: int, writes: bool):
        self.manager = manager
        self.entry = entry          # the order entry whose pools and state are used
        self.writes = writes        # False: this run reads another run's cache

    def pools(self):
        return self.manager.pools(self.entry)

    def block_table(self) -> torch.Tensor:
        return self.manager.block_table(self.entry)

    def state(self) -> torch.Tensor:
        return self.manager.state(self.entry)


class StepContext:
    def __init__(self, dtype: torch.dtype, device, buffers: Buffers, num_tokens: int, num_seqs: int,
                 token_ids, positions, token_rows, seq_starts, seq_rows, seq_first_pos, logit_index,
                 all_decode: bool, max_context: int, host_batch=None, num_sms: int = 148):
        self.dtype, self.device, self.buffers = dtype, device, buffers
        self.num_tokens, self.num_seqs = num_tokens, num_seqs
        self.token_ids, self.positions, self.token_rows = token_ids, positions, token_rows
        self.seq_starts, self.seq_rows, self.seq_first_pos = seq_starts, seq_rows, seq_first_pos
        self.logit_index = logit_index
        self.all_decode = all_decode        # every request brings exactly one token
        self.max_context = max_context      # upper bound of any request's length after this step
        self.host_batch = host_batch        # the host-side entries; None while a graph is recorded
        self.num_sms = num_sms

    # ------------------------------------------------------------------ kernel choice
    def gemm(self, out: torch.Tensor, x: torch.Tensor, w: torch.Tensor) -> None:
        """out = x w^T; out is [M, N] or float32 partial sums [S, M, N]."""
        ops.gemm_simt(out, x, w, splits=out.shape[0] if out.dim() == 3 else 1)

    def attention_partitions(self, num_kv_heads: int, page_size: int) -> int:
        """Into how many key partitions the SIMT attention splits each query.

        A function of static quantities only (batch width, limits), so that a recorded
        graph stays valid: enough blocks to fill the SMs twice, never more partitions
        than the longest row has pages.
        """
        blocks = max(1, num_kv_heads * self.num_tokens)
        want = -(-2 * self.num_sms // blocks)
        most = max(1, -(-self.max_context // (4 * page_size)))
        return max(1, min(want, most, 64))

    def attention(self, out, q, k_pool, v_pool, table, num_heads: int, scale: float, window: int) -> None:
        Hkv, page_size, D = k_pool.shape[1], k_pool.shape[2], k_pool.shape[3]
        NP = self.attention_partitions(Hkv, page_size)
        part_o = part_ml = None
        if NP > 1:
            N = q.shape[0]
            part_o = self.buffers.take_flat("attn_part_o", N * num_heads * NP * D, torch.float32)
            part_ml = self.buffers.take_flat("attn_part_ml", N * num_heads * NP * 2, torch.float32)
        ops.attention_simt(out, q, k_pool, v_pool, table, self.token_rows, self.positions, num_heads,
                           scale, window, NP, part_o, part_ml)
