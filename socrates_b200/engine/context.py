"""What a part sees of the step it runs in: the tokens, where they sit, and scratch.

A step is a flat batch of N tokens from R requests.  For token n the context gives
its id, its absolute position and the cache row of its request; for request r (in
batch order) the offset of its first token (`seq_starts`, R+1 entries), its cache row
and the position of its first token.  All of these are int32 device tensors that were
filled by one host-to-device copy before the step; no part reads anything back.
"""

from __future__ import annotations

import os
from typing import Dict, List, Optional, Tuple

import torch

from ..kernels import ops


def _l2_prefetch_budget() -> int:
    """Bytes of the next product's weights that a weight-streaming product asks for in L2 once
    its own loads are issued (`SOCRATES_L2_PREFETCH_MB`, 0 turns it off).  Measured on the 4B
    shape: 8 MB shortens a decode step at batch 8 by 1.8 %, 24 MB and more lengthen it."""
    return int(float(os.environ.get("SOCRATES_L2_PREFETCH_MB", "8")) * (1 << 20))


class Buffers:
    """Scratch tensors of the step, by name, with addresses that never change.

    `take(name, rows, shape, dtype)` returns the first `rows` rows of a buffer that is
    allocated once for `max_rows` rows, so a CUDA graph that recorded its address stays
    valid.  `take_wanted` does the same for buffers that hold one row per wanted logit
    (at most `max_wanted` rows: a generation step wants one row per request, far fewer
    than it has tokens, and a row of logits is as wide as the vocabulary).  `take_flat`
    serves buffers whose size does not scale with the row count; if one has to grow, the
    old storage is kept alive for the graphs that recorded it.
    """

    def __init__(self, max_rows: int, device, max_wanted: Optional[int] = None):
        self.max_rows = max_rows
        self.max_wanted = max_rows if max_wanted is None else max_wanted
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

    def take_wanted(self, name: str, rows: int, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        if rows > self.max_wanted:
            raise ValueError(f"{rows} wanted rows exceed the step limit of {self.max_wanted}")
        key = ("wanted:" + name, tuple(shape), dtype)
        buf = self._by_name.get(key)
        if buf is None:
            buf = torch.empty((self.max_wanted, *shape), dtype=dtype, device=self.device)
            self._by_name[key] = buf
        return buf[:rows]

    def take_flat(self, name: str, numel: int, dtype: torch.dtype, zeroed: bool = False) -> torch.Tensor:
        """`zeroed`: the storage is zero when it is allocated (for counters that kernels leave at
        zero after every use); it is not cleared again on later calls."""
        key = (name, dtype)
        buf = self._flat.get(key)
        if buf is None or buf.numel() < numel:
            if buf is not None:
                self._retired.append(buf)
            size = max(numel, 2 * buf.numel() if buf is not None else numel)
            buf = (torch.zeros if zeroed else torch.empty)(size, dtype=dtype, device=self.device)
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
                 all_decode: bool, max_context: int, host_batch=None, num_sms: int = 148,
                 status: Optional[torch.Tensor] = None, token_feedback: Optional[torch.Tensor] = None):
        self.dtype, self.device, self.buffers = dtype, device, buffers
        self.num_tokens, self.num_seqs = num_tokens, num_seqs
        self.token_ids, self.positions, self.token_rows = token_ids, positions, token_rows
        self.seq_starts, self.seq_rows, self.seq_first_pos = seq_starts, seq_rows, seq_first_pos
        self.logit_index = logit_index
        self.all_decode = all_decode        # every request brings exactly one token
        self.max_context = max_context      # upper bound of any request's length after this step
        self.host_batch = host_batch        # the host-side entries; None while a graph is recorded
        self.num_sms = num_sms
        self.status = status                # int32 device word the tensor-core kernels report to
        self.token_feedback = token_feedback   # int32 device tokens that ids -1 - j stand for (see ops.embed)
        self.weight_successor: Dict[int, torch.Tensor] = {}   # set by the model: address -> next weights
        self.l2_prefetch_bytes = _l2_prefetch_budget()

    # ------------------------------------------------------------------ kernel choice
    def uses_tensor_cores(self, x_dtype: torch.dtype, w: torch.Tensor) -> bool:
        """The tcgen05 kernel takes bfloat16 operands with 16-byte rows; everything else
        (the float32 engine, a matrix stored in float32, an odd K) runs on the CUDA cores."""
        return (x_dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] % 8 == 0
                and self.status is not None)

    def gemm_splits(self, M: int, w: torch.Tensor, x_dtype: torch.dtype, shares: bool = True) -> int:
        """Into how many K parts a product whose output is partial sums is cut.  `shares` = False:
        the caller would rather have one part in the model dtype than the float32 parts of the
        equal-shares kernel (whose gain the wider output would eat).

        The weight-streaming regime (M <= 64) is cut into enough blocks to keep two resident
        on every SM, at least two K blocks of 64 each; a product with many rows only where its
        tiles would leave more than half of the SMs idle.  A function of the shapes alone, so a
        recorded graph stays valid.
        """
        if not self.uses_tensor_cores(x_dtype, w):
            return 1
        N, K = w.shape
        if M > 64:
            parts = self.gemm_shares(M, w, x_dtype) if shares else 0
            if parts:
                return parts
            # Many rows but few tiles (a short prompt portion through a narrow projection): cut K
            # so that the tiles cover the SMs.  Measured on the 4B shape at 512 rows: o 29 -> 20 us,
            # down 57 -> 33 us with three parts; from 1,024 rows on a cut no longer pays.
            tiles = -(-M // 128) * -(-N // 256)
            if 2 * tiles > self.num_sms:
                return 1
            return ops.gemm_tcgen05_splits(K, max(1, min(4, self.num_sms // tiles, (-(-K // 64)) // 8)))
        tiles = -(-N // 128)
        want = max(1, (2 * self.num_sms) // tiles)
        most = max(1, (-(-K // 64)) // 2)
        return ops.gemm_tcgen05_splits(K, min(want, most, 16))

    def gemm_shares(self, M: int, w: torch.Tensor, x_dtype: torch.dtype) -> int:
        """Parts of the pair kernel in equal shares of K blocks if a product of M rows whose output
        is partial sums should run on it, else 0.  Whole tiles run in waves over the SMs; a product
        whose last wave is mostly empty (a 2,048-row portion through a 2,560-wide projection: 80
        tiles of 256 x 256 for 74 pairs, 256 tiles of 128 x 160 for 148 SMs) loses up to half of
        its time there.  Chosen when the model of the kernels' measured costs per K block (690
        clocks for a pair's 256 x 256 tile; 540 + 0.94 * width for one SM's 128 x width tile) says
        that equal shares take less than 0.9 of the best whole-tile choice, and both operands
        together stay well inside the L2 cache (96 MB): whole tiles run the row tiles of a weight
        panel side by side, so the panel comes from memory once, while equal shares shift every
        pair to another K offset and rely on the cache to keep what an earlier pair fetched
        (measured at 2,048 rows: 2,560 x 9,728, 90 MB of operands, 94 against 116 us; 5,120 x
        25,600, 367 MB, 525 against 469 us).  Shapes alone decide."""
        if not self.uses_tensor_cores(x_dtype, w) or os.environ.get("SOCRATES_GEMM_SHARES", "1") == "0":
            return 0
        N, K = w.shape
        if (M + N) * K * 2 > 96 * (1 << 20):
            return 0
        parts = ops.gemm_tcgen05_shares_parts(M, N, K)
        if parts == 0:
            return 0
        pairs = max(1, self.num_sms // 2)
        shares_cost = (-(-M // 256) * -(-N // 256)) * 690.0 / pairs
        rows128 = -(-M // 128)
        whole_cost = min((-(-(rows128 * -(-N // bn)) // self.num_sms)) * (540.0 + 0.94 * bn) for bn in (256, 160, 128))
        if M >= 4096:       # the pair kernel with whole tiles is the choice there
            whole_cost = min(whole_cost, (-(-(-(-M // 256) * -(-N // 256)) // pairs)) * 690.0)
        return parts if shares_cost < 0.9 * whole_cost else 0

    def can_fuse_silu_mul(self, M: int, w: torch.Tensor, x_dtype: torch.dtype) -> bool:
        """Whether the product with an interleaved gate/up matrix can apply SiLU*mul in its
        epilogue (the tensor-core kernels do, for few rows and for many)."""
        return self.uses_tensor_cores(x_dtype, w) and w.shape[0] % 2 == 0 and (M <= 64 or w.shape[0] >= 128)

    def gemm(self, out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, epilogue: int = 0) -> None:
        """out = x w^T; out is [M, N] or float32 partial sums [S, M, N]; with epilogue 1 (see
        can_fuse_silu_mul) out is [M, N/2] = up * silu(gate) of interleaved columns."""
        S = out.shape[0] if out.dim() == 3 else 1
        if self.uses_tensor_cores(x.dtype, w):
            M = x.shape[0]
            if M > 64 and out.dim() == 3 and epilogue == 0 and S == self.gemm_shares(M, w, x.dtype) and S > 0:
                ops.gemm_tcgen05(out, x, w, self.status, S, variant=ops.SHARES_VARIANT)
                return
            ops.gemm_tcgen05(out if out.dim() == 3 and S > 1 else out.view(out.shape[-2], out.shape[-1]),
                             x, w, self.status, S, epilogue=epilogue, prefetch=self._next_weights(w))
        else:
            if epilogue:
                raise ValueError("the fused epilogue exists only in the tensor-core kernel")
            ops.gemm_simt(out, x, w, splits=S)

    def _next_weights(self, w: torch.Tensor):
        nxt = self.weight_successor.get(w.data_ptr())
        if nxt is None or self.l2_prefetch_bytes <= 0 or not nxt.is_contiguous():
            return None
        return (nxt, self.l2_prefetch_bytes)
