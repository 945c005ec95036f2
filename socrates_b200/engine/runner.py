"""The step function: one batch of (request, its next tokens) through the model.

`ModelRunner.step(entries)` runs only the tokens it is given, as one flat batch, from
the cache that earlier steps left, and returns float32 logits at the wanted places.
Portions of prompts and single decode tokens mix freely and a prompt may be cut
anywhere.  The reference's forward takes a rectangle instead, either one whole prompt
or n rows of one token (model/qwen/qwen_kv_paged.py:207-224).

Host and device: the step's integers are written into one pinned buffer and reach the
device in one copy; nothing is read back inside the step.  A step in which every
request brings one token is recorded once per batch width into a CUDA graph and
replayed afterwards (the reference compiles one graph per width with
torch.compile(mode="reduce-overhead"), model/inference_paged.py:99-130).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..cache.manager import CacheManager
from ..kernels import ops
from ..kernels.library import Counters
from .context import Buffers, StepContext
from .model import Model


@dataclass
class StepEntry:
    """The next tokens of one request: `tokens` start at position `start` of cache row
    `row`; `want` lists the places among these tokens whose logits are asked for."""
    row: int
    tokens: Sequence[int]
    start: int
    want: Sequence[int] = ()


@dataclass
class SamplingArgs:
    """How to turn one wanted row of logits into a token (see socrates_b200.sampling)."""
    temperature: float = 0.0
    seed: int = 0
    counter: int = 0


@dataclass
class StepResult:
    logits: Optional[torch.Tensor]          # float32 [wanted, vocab] on the device, or None
    tokens: Optional[torch.Tensor] = None   # int32 [wanted] on the device when sampling was asked for
    num_tokens: int = 0


class _Layout:
    """Offsets of the step's integer arrays inside the staging buffer."""

    def __init__(self, T: int, R: int):
        self.T, self.R = T, R
        self.ids, self.pos, self.rows, self.logit = 0, T, 2 * T, 3 * T
        self.temp, self.seed, self.counter = 4 * T, 5 * T, 6 * T
        self.seq_starts = 7 * T
        self.seq_rows = self.seq_starts + R + 1
        self.seq_first = self.seq_rows + R
        self.total = self.seq_first + R


class ModelRunner:
    def __init__(self, model: Model, cache: CacheManager, dtype: torch.dtype, device,
                 max_tokens: int, max_seqs: int, use_graphs: bool = True, max_wanted: Optional[int] = None):
        """`max_wanted`: the most logits rows one step may ask for (default: one per token, which
        trace replay needs; generation wants one per request and passes max_seqs)."""
        self.model, self.cache = model, cache
        self.dtype, self.device = dtype, torch.device(device)
        self.max_tokens, self.max_seqs = max_tokens, max_seqs
        self.max_wanted = max_tokens if max_wanted is None else min(max_wanted, max_tokens)
        self.vocab = model.plan.vocab_size
        self.buffers = Buffers(max_tokens, self.device, self.max_wanted)
        self.layout = _Layout(max_tokens, max_seqs)
        self.dev_meta = torch.zeros(self.layout.total, dtype=torch.int32, device=self.device)
        self._staging = [[torch.zeros(self.layout.total, dtype=torch.int32).pin_memory(), None]
                         for _ in range(4)]
        self._staging_np = [b.numpy() for b, _ in self._staging]
        self._staging_f32 = [b.view(torch.float32).numpy() for b, _ in self._staging]
        self._next = 0
        # sampled tokens and the kernels' status word share one buffer, so that a step's
        # read-back is one copy: [status, token 0, token 1, ...]
        self._readback = torch.zeros(max_tokens + 1, dtype=torch.int32, device=self.device)
        self.status = self._readback[0:1]
        self.sampled = self._readback[1:]
        self._events = [torch.cuda.Event() for _ in self._staging]
        # read-backs in flight: pinned copies of [status, tokens...], one slot per step that may be
        # launched before an earlier one's tokens are read
        self._rb_host = [torch.zeros(max_tokens + 1, dtype=torch.int32).pin_memory() for _ in range(3)]
        self._rb_np = [b.numpy() for b in self._rb_host]
        self._rb_events = [torch.cuda.Event() for _ in self._rb_host]
        self._rb_next = 0
        self.sample_scratch = torch.zeros(ops.sample_scratch_size(max_tokens, self.vocab), dtype=torch.int32,
                                          device=self.device)
        self.use_graphs = use_graphs and model.supports_graph
        self._graphs: Dict[Tuple[int, int, bool], Tuple[torch.cuda.CUDAGraph, Optional[torch.Tensor]]] = {}
        self._eager_decode_done: set = set()
        self.num_sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.steps_run = 0
        self.graph_replays = 0
        self.kernel_launches = 0    # kernels launched by steps, replays of recorded graphs included
        self._graph_kernels: Dict[Tuple[int, bool], int] = {}

    # ------------------------------------------------------------------ staging
    def _stage(self) -> Tuple[torch.Tensor, int]:
        i = self._next
        self._next = (i + 1) % len(self._staging)
        buf, ev = self._staging[i]
        if ev is not None:
            ev.synchronize()
        return buf, i

    def _fill(self, entries: Sequence[StepEntry], sampling, ahead: int = 0) -> Tuple[int, int, int, bool, int]:
        L = self.layout
        if not entries:
            raise ValueError("a step needs at least one entry")
        if len(entries) > self.max_seqs:
            raise ValueError(f"{len(entries)} requests exceed the step limit of {self.max_seqs}")
        ids: List[int] = []
        pos: List[int] = []
        rows: List[int] = []
        logit: List[int] = []
        starts = [0]
        seen = set()
        all_decode = True
        max_ctx = 0
        for e in entries:
            n = len(e.tokens)
            if n < 1:
                raise ValueError("an entry needs at least one token")
            if e.row in seen:
                raise ValueError(f"row {e.row} appears twice in one step")
            seen.add(e.row)
            if not 0 <= e.row < self.cache.max_rows:
                raise ValueError(f"row {e.row} is outside the cache")
            if e.start != self.cache.lengths[e.row] + ahead:
                raise ValueError(f"row {e.row} holds {self.cache.lengths[e.row]} tokens; "
                                 f"the entry starts at {e.start}")
            if e.start + n > self.cache.max_len:
                raise ValueError(f"row {e.row} would exceed {self.cache.max_len} tokens")
            for t in e.tokens:
                if not -self.max_tokens <= t < self.vocab:      # -1 - j: the previous step's j-th sample
                    raise ValueError(f"token id {t} is outside the vocabulary of {self.vocab}")
            base = len(ids)
            ids.extend(int(t) for t in e.tokens)
            pos.extend(range(e.start, e.start + n))
            rows.extend([e.row] * n)
            for w in e.want:
                if not 0 <= w < n:
                    raise ValueError(f"wanted place {w} is outside the entry's {n} tokens")
                logit.append(base + w)
            starts.append(len(ids))
            all_decode &= n == 1
            max_ctx = max(max_ctx, e.start + n)
        N, M, R = len(ids), len(logit), len(entries)
        if N > self.max_tokens:
            raise ValueError(f"{N} tokens exceed the step limit of {self.max_tokens}")
        if M > self.max_wanted:
            raise ValueError(f"{M} wanted logits exceed the step limit of {self.max_wanted}")
        if sampling is not None and len(sampling) != M:
            raise ValueError(f"{len(sampling)} sampling entries for {M} wanted logits")

        buf, slot = self._stage()
        nb = self._staging_np[slot]                 # numpy view of the pinned buffer: cheap list assignment
        nb[L.ids:L.ids + N] = ids
        nb[L.pos:L.pos + N] = pos
        nb[L.rows:L.rows + N] = rows
        if M:
            nb[L.logit:L.logit + M] = logit
        if sampling is not None and M:
            self._staging_f32[slot][L.temp:L.temp + M] = [s.temperature for s in sampling]
            nb[L.seed:L.seed + M] = [_as_i32(s.seed) for s in sampling]
            nb[L.counter:L.counter + M] = [_as_i32(s.counter) for s in sampling]
        nb[L.seq_starts:L.seq_starts + R + 1] = starts
        nb[L.seq_rows:L.seq_rows + R] = [e.row for e in entries]
        nb[L.seq_first:L.seq_first + R] = [e.start for e in entries]
        self.dev_meta.copy_(buf, non_blocking=True)     # the step's one host-to-device copy
        ev = self._events[slot]
        ev.record()
        self._staging[slot][1] = ev
        return N, M, R, all_decode, max_ctx

    def _context(self, N: int, M: int, R: int, all_decode: bool, max_ctx: int, host_batch) -> StepContext:
        L, m = self.layout, self.dev_meta
        return StepContext(
            self.dtype, self.device, self.buffers, N, R,
            token_ids=m[L.ids:L.ids + N], positions=m[L.pos:L.pos + N], token_rows=m[L.rows:L.rows + N],
            seq_starts=m[L.seq_starts:L.seq_starts + R + 1], seq_rows=m[L.seq_rows:L.seq_rows + R],
            seq_first_pos=m[L.seq_first:L.seq_first + R],
            logit_index=m[L.logit:L.logit + M] if M else None,
            all_decode=all_decode, max_context=max_ctx, host_batch=host_batch, num_sms=self.num_sms,
            status=self.status, token_feedback=self.sampled)

    def begin_read(self, count: int) -> Tuple[int, int]:
        """Start the copy of the `count` tokens the last step sampled (and of the kernels'
        status word) to the host; `finish_read` waits for it.  A later step may be launched in
        between: the copy is ordered before it on the stream."""
        slot = self._rb_next
        self._rb_next = (slot + 1) % len(self._rb_host)
        self._rb_host[slot][:count + 1].copy_(self._readback[:count + 1], non_blocking=True)
        self._rb_events[slot].record()
        return slot, count

    def finish_read(self, handle: Tuple[int, int]) -> List[int]:
        slot, count = handle
        self._rb_events[slot].synchronize()
        host = self._rb_np[slot][:count + 1].tolist()
        if host[0] != 0:
            self.status.zero_()
            raise RuntimeError(f"a tensor-core kernel gave up waiting on its pipeline (code {host[0]}); "
                               f"the step's results are not valid")
        return host[1:]

    def read_tokens(self, count: int) -> List[int]:
        """The `count` tokens the last step sampled, as a host list, and a check of the
        kernels' status word, in ONE device-to-host copy (which also waits for the step)."""
        return self.finish_read(self.begin_read(count))

    @torch.no_grad()
    def warmup(self, max_width: int, sample: bool = True) -> int:
        """Record the decode graph of every batch width 1..max_width before serving, as the
        reference does at start-up (model/inference_paged.py:110-130).  The steps run on rows
        that own no page, so everything they write lands in the null page.  Returns the
        number of graphs recorded."""
        if not self.use_graphs:
            return 0
        L, made = self.layout, 0
        for n in range(1, min(max_width, self.max_seqs, self.cache.max_rows) + 1):
            key = (n, sample)
            if key in self._graphs:
                continue
            buf, slot = self._stage()
            nb = self._staging_np[slot]
            nb[:] = 0
            nb[L.rows:L.rows + n] = list(range(n))
            nb[L.logit:L.logit + n] = list(range(n))
            nb[L.seq_starts:L.seq_starts + n + 1] = list(range(n + 1))
            nb[L.seq_rows:L.seq_rows + n] = list(range(n))
            self.dev_meta.copy_(buf, non_blocking=True)
            ev = self._events[slot]
            ev.record()
            self._staging[slot][1] = ev
            ctx = self._context(n, n, n, True, self.cache.max_len, None)
            self._run(ctx, n, sample)                       # loads every kernel, sizes every buffer
            graph = torch.cuda.CUDAGraph()
            before = Counters.launches
            with torch.cuda.graph(graph):
                logits, tokens = self._run(ctx, n, sample)
            self._graph_kernels[key] = Counters.launches - before
            self._graphs[key] = (graph, logits, tokens)
            self._eager_decode_done.add(key)
            made += 1
        torch.cuda.synchronize()
        return made

    def check_status(self) -> None:
        """Raise if a kernel reported that one of its bounded waits gave up.  Reads one
        word back, so call it where the host synchronises anyway (after a step's tokens
        or logits were read)."""
        code = int(self.status.item())
        if code != 0:
            self.status.zero_()
            raise RuntimeError(f"a tensor-core kernel gave up waiting on its pipeline (code {code}); "
                               f"the step's results are not valid")

    def _run(self, ctx: StepContext, M: int, sample: bool):
        with ops.stream_scope():            # one stream look-up for the step's kernels (also while a graph records)
            logits = self.model.forward(ctx, self.cache)
            tokens = None
            if sample and M:
                L, m = self.layout, self.dev_meta
                tokens = self.sampled[:M]
                ops.sample(tokens, logits, m[L.temp:L.temp + M].view(torch.float32),
                           m[L.seed:L.seed + M], m[L.counter:L.counter + M], self.sample_scratch)
        return logits, tokens

    def prepare(self, entries: Sequence[StepEntry],
                sampling: Optional[Sequence[SamplingArgs]] = None) -> StepContext:
        """Copy the step's integers to the device and return the context the parts see.
        `step` does this itself; tests of single parts call it to run a part alone."""
        self.cache.flush()
        N, M, R, all_decode, max_ctx = self._fill(entries, sampling)
        return self._context(N, M, R, all_decode, max_ctx, entries)

    # ------------------------------------------------------------------ the step
    @torch.no_grad()
    def step(self, entries: Sequence[StepEntry],
             sampling: Optional[Sequence[SamplingArgs]] = None, ahead: int = 0) -> StepResult:
        """Run one batch.  The caller has reserved pages for every entry
        (`cache.reserve(row, start + len(tokens))`) and commits the new lengths after.
        `ahead` = 1: the step is launched before the one before it is committed, so every entry
        starts one past its row's committed length (and may name its token as -1 - j, the j-th
        token the step before sampled)."""
        self.cache.flush()
        N, M, R, all_decode, max_ctx = self._fill(entries, sampling, ahead)
        sample = sampling is not None
        self.steps_run += 1
        if self.use_graphs and all_decode and M == N:
            key = (N, sample)
            if key not in self._graphs and key in self._eager_decode_done:
                ctx = self._context(N, M, R, True, self.cache.max_len, None)
                graph = torch.cuda.CUDAGraph()
                before = Counters.launches
                with torch.cuda.graph(graph):
                    logits, tokens = self._run(ctx, M, sample)
                self._graph_kernels[key] = Counters.launches - before
                self._graphs[key] = (graph, logits, tokens)
            if key in self._graphs:
                graph, logits, tokens = self._graphs[key]
                graph.replay()
                self.graph_replays += 1
                self.kernel_launches += self._graph_kernels[key]
                return StepResult(logits, tokens, N)
            self._eager_decode_done.add(key)
            max_ctx = self.cache.max_len     # the same launch shapes the graph will record
        ctx = self._context(N, M, R, all_decode, max_ctx, entries)
        before = Counters.launches
        logits, tokens = self._run(ctx, M, sample)
        self.kernel_launches += Counters.launches - before
        return StepResult(logits, tokens, N)


def _as_i32(x: int) -> int:
    x &= 0xFFFFFFFF
    return x - (1 << 32) if x >= (1 << 31) else x
