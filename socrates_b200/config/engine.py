"""Limits of one engine instance: rows, context, pages, token budget.

The reference keeps these as module constants (model/inference_cont.py:21-24:
MAX_BATCH=18, MAX_NEW_TOKENS=1024, MAX_LEN=2048, MAX_QUEUE=16*MAX_BATCH) and
KV_BLOCK=16 (model/inference_paged.py:51).  The names of the reference's Engine
arguments (max_batch, max_len, max_new_tokens, block_size, num_blocks) are kept.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass
class EngineConfig:
    max_batch: int = 64               # live requests (cache rows)
    max_len: int = 8192               # tokens one row may hold
    max_new_tokens: int = 1024
    block_size: int = 16              # slots per page
    num_blocks: Optional[int] = None  # pages per cache group; None = from free memory (see pages_from_memory)
    kv_memory_fraction: float = 0.9   # share of the memory left after the weights that pages may take
    token_budget: int = 2048          # most tokens one step runs
    max_queue: Optional[int] = None   # None = 16 * max_batch
    dtype: str = "bfloat16"           # "bfloat16" or "float32"
    compile: bool = True              # one CUDA graph per decode batch width

    def validate(self) -> None:
        if self.max_batch < 1:
            raise ValueError("max_batch must be at least 1")
        if self.block_size < 1 or self.block_size & (self.block_size - 1):
            raise ValueError(f"block_size={self.block_size} must be a power of two")
        if self.max_len < 1:
            raise ValueError("max_len must be positive")
        if self.token_budget < 1:
            raise ValueError("token_budget must be at least 1")
        if self.dtype not in ("bfloat16", "float32"):
            raise ValueError(f"dtype must be 'bfloat16' or 'float32', not {self.dtype!r}")
        if self.num_blocks is not None and self.num_blocks < 1:
            raise ValueError("num_blocks must be at least 1")
        if not 0.0 < self.kv_memory_fraction <= 1.0:
            raise ValueError("kv_memory_fraction must be in (0, 1]")

    @property
    def blocks_per_row(self) -> int:
        return -(-self.max_len // self.block_size)

    @property
    def queue_limit(self) -> int:
        return self.max_queue if self.max_queue is not None else 16 * self.max_batch

    @property
    def pool_blocks(self) -> int:
        """Pages per group when nothing limits them: every row at its full length, which is
        the reference's rule (model/inference_paged.py:83-84)."""
        return self.num_blocks if self.num_blocks is not None else self.max_batch * self.blocks_per_row

    def pages_from_memory(self, free_bytes: int, bytes_per_page: int) -> int:
        """Pages per group for `num_blocks=None`: what `kv_memory_fraction` of the memory that
        is free once the weights are loaded pays for, never more than every row at full length
        would use, never fewer than one row needs.  Pages are taken lazily and the scheduler
        preempts when they run out, so a pool smaller than rows x max_len is safe."""
        if self.num_blocks is not None:
            return self.num_blocks
        afford = int(free_bytes * self.kv_memory_fraction) // max(1, bytes_per_page)
        return max(self.blocks_per_row, min(self.max_batch * self.blocks_per_row, afford))
