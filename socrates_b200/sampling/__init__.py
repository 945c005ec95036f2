"""Sampling: greedy and temperature.

The reference samples greedily only: `logits[:, -1].argmax(-1)` on the host side of
the step (model/inference_paged.py:166,193), ties to the lowest index; temperature is
described as softmax(logits / T) (docs/day_1_docs.md:45-52) and forced to 0 in its
benchmark.  Here both run in one kernel on float32 logits (socrates_b200/csrc/sampling.cu):

* temperature 0: argmax, ties to the lowest index;
* temperature T > 0: a draw from softmax(logits / T) by the Gumbel-max rule,
  token = argmax_i (logit_i / T - log(-log u_i)).

u_i is a counter-based uniform, a pure function of (seed, counter, i): with mix32 the
three-round xorshift-multiply finalizer (constants 0x7FEB352D, 0x846CA68B, shifts
16/15/16) on unsigned 32-bit integers,

    key = mix32(mix32(seed ^ 0x9E3779B9) ^ mix32(counter + 0x85EBCA6B))
    u_i = ((mix32((i + 0x165667B1) ^ key) >> 9) + 0.5) / 2^23

`counter` is the number of tokens the request has produced so far, so a request's
tokens depend on its seed alone: not on the batch it ran in, not on how its prompt was
cut, not on whether it was preempted and recomputed.
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0     # 0 = greedy
    seed: int = 0

    def validate(self) -> None:
        if not self.temperature >= 0.0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")


__all__ = ["SamplingParams"]
