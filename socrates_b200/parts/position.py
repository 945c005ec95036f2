"""Position encodings as data for the mixer's rotation kernel.

A position encoding hands the mixer a float32 table `inv_freq[rotary_dim/2]` and the
number of leading dims that rotate; the kernel computes angle = float32(position) *
inv_freq[j] and pairs dim j with j + rotary_dim/2.  Keys are stored rotated, so
positions are absolute and nothing else in the engine knows about the encoding.
Another encoding (a fraction of the dims, scaled frequencies, none at all) is another
table: register a class with `tables()`.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from .base import Part, register_part


class Rotary(Part):
    """inv_freq_j = theta^(-2j/D), j < D/2, in float32 exactly as the reference builds
    it (model/qwen/qwen_kv_cont.py:56-64)."""

    def __init__(self, spec, name=""):
        super().__init__(spec, name)
        self.head_dim = int(spec.params["head_dim"])
        self.rotary_dim = int(spec.params.get("rotary_dim", self.head_dim))
        self.theta = float(spec.params["theta"])
        if self.rotary_dim % 2 or not 0 <= self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        self._table: Optional[torch.Tensor] = None

    def inv_freq(self) -> torch.Tensor:
        r = self.rotary_dim
        return 1.0 / (self.theta ** (torch.arange(0, r, 2).float() / r))

    def tables(self, device) -> Tuple[torch.Tensor, int]:
        if self._table is None or self._table.device != torch.device(device):
            t = self.inv_freq() if self.rotary_dim else torch.zeros(1)
            self._table = t.to(device=device, dtype=torch.float32).contiguous()
        return self._table, self.rotary_dim


class NoPosition(Part):
    """No rotation: the mixer's kernel passes every dim through."""

    def __init__(self, spec, name=""):
        super().__init__(spec, name)
        self._table = None

    def tables(self, device):
        if self._table is None:
            self._table = torch.zeros(1, dtype=torch.float32, device=device)
        return self._table, 0


register_part("position", "rotary", Rotary)
register_part("position", "none", NoPosition)
