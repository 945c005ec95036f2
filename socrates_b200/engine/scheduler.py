"""The scheduler: admits requests, cuts prompts into portions under a token budget,
decodes, finishes and frees.  Host code only; it decides, the runner computes.

The reference's loop (model/inference_paged.py:132-237) is submit -> admit (reserve the
worst case, prefill the whole prompt alone) -> sweep -> decode_step (all live rows,
one token) -> sweep, with rows kept packed at 0..n-1 by moving the last row into a
retired row's place.  Kept from it: FIFO admission, the QueueFull / TooLong guards at
the door, the stop rule (a stop token is not appended; at most max_new_tokens are),
the cancelled flag, retire + compaction + refill in the same iteration.  Changed:

* **One kind of step.**  Every live request contributes its next tokens: one token if
  it is decoding, a portion of its prompt otherwise.  Decoding requests come first,
  then prompt portions fill what is left of `token_budget`.  Several prompts may share
  a step, and a prompt is cut wherever the budget ends.  A waiting request is admitted
  only while the pool has pages for its first portion and one to spare for each live
  request (see `_room_to_admit`).
* **Pages on demand.**  A request takes pages for the tokens of this step only.
* **When pages run out** (decided here, tested in tests/test_scheduler.py): a request
  that cannot get its pages makes the most recently admitted *other* live request give
  up all of its pages and go back to the front of the queue; when it is admitted again
  its prompt and the tokens it had produced are recomputed, and sampling continues
  with the same counters, so its output is unchanged.  If the request that lacks pages
  is itself the most recently admitted, it waits for this step (a prompt portion is
  first shrunk to the pages that are free).  The oldest request can therefore always
  proceed, and `submit` refuses requests that could not fit the pool alone.
"""

from __future__ import annotations

import queue
import threading
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, List, Optional, Sequence

from ..cache.allocator import pages_for
from ..sampling import SamplingParams


class QueueFull(Exception):
    """Too many requests are waiting (model/inference_paged.py:133-134)."""


class TooLong(Exception):
    """Prompt plus new tokens exceed a row or the page pool (model/inference_paged.py:144-146)."""


@dataclass
class Request:
    """One generation request; field names follow the reference's Request
    (model/inference_cont.py:65-82) where it has them."""
    ids: List[int]                                   # prompt token ids
    max_new_tokens: int
    sampling: SamplingParams = field(default_factory=SamplingParams)
    prompt: Optional[str] = None
    output: List[int] = field(default_factory=list)
    done: bool = False
    row: int = -1
    cancelled: bool = False
    submitted: float = field(default_factory=time.perf_counter)
    admitted: float = 0.0
    first_token: float = 0.0
    finished: float = 0.0
    event: threading.Event = field(default_factory=threading.Event)
    # a queue that receives every produced token and None at the end (the reference's req.stream,
    # model/inference_paged.py:136-138, 196-198, is an asyncio queue fed from the serve thread; this
    # one is thread-safe and needs no event loop)
    stream: Optional["queue.Queue"] = None
    # scheduler state
    cached: int = 0            # tokens of ids + output that are in the cache
    preemptions: int = 0
    order: int = -1            # admission counter; larger = admitted later

    @property
    def sequence_len(self) -> int:
        return len(self.ids) + len(self.output)

    def token_at(self, i: int) -> int:
        n = len(self.ids)
        return self.ids[i] if i < n else self.output[i - n]


@dataclass
class PlannedEntry:
    request: Request
    row: int
    start: int
    count: int
    samples: bool              # the portion reaches the end of what is known: a token is drawn


@dataclass
class StepPlan:
    entries: List[PlannedEntry]
    preempted: List[Request] = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return sum(e.count for e in self.entries)


class Scheduler:
    def __init__(self, cache, max_batch: int, max_len: int, token_budget: int, max_queue: int,
                 stop_ids: Sequence[int] = ()):
        if token_budget < max_batch:
            raise ValueError(f"token_budget={token_budget} must cover one token for each of "
                             f"max_batch={max_batch} rows")
        self.cache = cache
        self.max_batch, self.max_len = max_batch, max_len
        self.token_budget, self.max_queue = token_budget, max_queue
        self.stop_ids = frozenset(int(s) for s in stop_ids)
        self.pending: Deque[Request] = deque()
        self.rows: List[Optional[Request]] = [None] * max_batch
        self.n_active = 0
        self._admissions = 0
        self.prompt_tokens = 0       # counters, as socrates_prompt_tokens_total /
        self.output_tokens = 0       # socrates_output_tokens_total (model/inference_cont.py:32-33)
        self.preemptions = 0

    # ------------------------------------------------------------------ the door
    def submit(self, req: Request) -> Request:
        if len(self.pending) >= self.max_queue:
            raise QueueFull(f"{len(self.pending)} requests already waiting")
        if not req.ids:
            raise ValueError("a prompt needs at least one token")
        if req.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be at least 1")
        total = len(req.ids) + req.max_new_tokens
        if total > self.max_len:
            raise TooLong(f"prompt is {len(req.ids)} tokens; with {req.max_new_tokens} new it "
                          f"exceeds the {self.max_len}-token row")
        for g in self.cache.groups:
            need = pages_for(total, self.cache.page_size)
            if g.spec.window is not None:
                # a windowed group holds the window and the token being written, which may
                # straddle one page edge more than their count fills
                need = min(need, pages_for(g.spec.window + 1, self.cache.page_size) + 1)
            if need > g.allocator.num_pages:
                raise TooLong(f"{total} tokens need {need} pages at once; the pool has {g.allocator.num_pages}")
        req.sampling.validate()
        self.pending.append(req)
        return req

    @property
    def live(self) -> List[Request]:
        return [r for r in self.rows[:self.n_active] if r is not None]

    def has_work(self) -> bool:
        return bool(self.pending) or self.n_active > 0

    # ------------------------------------------------------------------ rows
    def _admit(self, req: Request) -> None:
        row = self.n_active
        self.cache.assign(row)
        self.rows[row] = req
        req.row = row
        req.cached = 0
        req.order = self._admissions
        self._admissions += 1
        if not req.admitted:
            req.admitted = time.perf_counter()
        self.n_active += 1

    def _vacate(self, req: Request) -> None:
        """Free the request's row and keep live rows packed at 0..n_active-1
        (model/inference_paged.py:213-225)."""
        row, last = req.row, self.n_active - 1
        self.cache.release(row)
        if row != last:
            self.cache.move_row(last, row)
            self.rows[row] = self.rows[last]
            self.rows[row].row = row
        self.rows[last] = None
        self.n_active -= 1
        req.row = -1

    @staticmethod
    def _drop(req: Request) -> None:
        """A request that was cancelled before it got a row."""
        if req.stream is not None:
            req.stream.put(None)
        req.event.set()

    def retire(self, req: Request) -> None:
        self._vacate(req)
        if not req.finished:
            req.finished = time.perf_counter()
        if req.stream is not None:
            req.stream.put(None)            # the end of the stream, for a finished and for a cancelled request
        req.event.set()

    def preempt(self, req: Request) -> None:
        self._vacate(req)
        req.cached = 0
        req.preemptions += 1
        self.preemptions += 1
        self.pending.appendleft(req)

    def sweep(self) -> None:
        for req in [r for r in self.live if r.done or r.cancelled]:
            self.retire(req)

    # ------------------------------------------------------------------ planning
    def _latest_other(self, req: Request, protected) -> Optional[Request]:
        others = [r for r in self.live if r is not req and r not in protected]
        return max(others, key=lambda r: r.order) if others else None

    def _reserve(self, req: Request, new_len: int, planned: List[PlannedEntry],
                 preempted: List[Request]) -> bool:
        """Get pages for `req` to reach `new_len`, preempting later requests if needed."""
        while not self.cache.reserve(req.row, new_len):
            protected = [e.request for e in planned]
            victim = self._latest_other(req, protected)
            if victim is None or victim.order < req.order:
                return False
            self.preempt(victim)
            preempted.append(victim)
        return True

    def plan(self) -> Optional[StepPlan]:
        """Decide the next step.  Reserves the pages it needs; returns None when there
        is nothing to run.

        Live requests are served oldest first, so that whoever lacks pages takes them
        from requests admitted after it and the oldest request always proceeds.  One
        token of the budget is set aside for every decoding request before any prompt
        portion is sized; in the batch the decode tokens come first.
        """
        while self.pending and self.pending[0].cancelled:
            self._drop(self.pending.popleft())
        self.sweep()
        planned: List[PlannedEntry] = []
        preempted: List[Request] = []
        by_age = sorted(self.live, key=lambda r: r.order)
        n_decode = sum(1 for r in by_age if r.sequence_len - r.cached == 1)
        prefill_budget = self.token_budget - n_decode

        for req in by_age:
            if req.row < 0:
                continue                                    # preempted earlier in this pass
            if req.sequence_len - req.cached == 1:
                if self._reserve(req, req.cached + 1, planned, preempted):
                    planned.append(PlannedEntry(req, req.row, req.cached, 1, True))
            elif prefill_budget >= 1:
                prefill_budget -= self._plan_portion(req, prefill_budget, planned, preempted)

        # admissions, FIFO, while a row and budget are left
        while self.pending and self.n_active < self.max_batch and prefill_budget >= 1:
            req = self.pending[0]
            if req.cancelled:
                self._drop(self.pending.popleft())
                continue
            if req in preempted:
                break                       # it just gave up its pages: not in this step
            if not self._room_to_admit(req, prefill_budget):
                break                       # it would only take pages that the live requests need next
            self.pending.popleft()
            self._admit(req)
            prefill_budget -= self._plan_portion(req, prefill_budget, planned, preempted)

        if not planned:
            return None
        planned.sort(key=lambda e: 0 if e.count == 1 and e.samples else 1)   # stable: decode tokens first
        for e in planned:
            e.row = e.request.row           # compaction after a preemption may have moved rows
        return StepPlan(planned, preempted)

    def _room_to_admit(self, req: Request, budget: int) -> bool:
        """Whether admitting `req` now is worth a row.  With nobody live it always is (the oldest
        request must proceed, if only with a shrunk portion).  Otherwise every group must have free
        pages for its first portion AND one page to spare for each live request: a request admitted
        into the last free pages is the newest one, so the next live request that needs a page
        would take them straight back and the portion would have been computed for nothing
        (measured at real widths with a pool a twentieth of the demand: 398 preemptions for 150
        requests before this rule)."""
        if self.n_active == 0:
            return self.cache.can_reserve(self.n_active, 1)
        first = min(req.sequence_len, budget)
        need = pages_for(first, self.cache.page_size) + self.n_active
        return all(g.allocator.n_free >= min(need, g.allocator.num_pages) for g in self.cache.groups)

    def _plan_portion(self, req: Request, budget: int, planned: List[PlannedEntry],
                      preempted: List[Request]) -> int:
        """Plan the next portion of `req` under `budget` tokens; returns its size (0: it waits)."""
        count = min(req.sequence_len - req.cached, budget)
        if count < 1:
            return 0
        if not self._reserve(req, req.cached + count, planned, preempted):
            count = min(count, self._tokens_that_fit(req))      # shrink to the pages that are free
            if count < 1 or not self.cache.reserve(req.row, req.cached + count):
                return 0
        planned.append(PlannedEntry(req, req.row, req.cached, count,
                                    req.cached + count == req.sequence_len))
        return count

    def _tokens_that_fit(self, req: Request) -> int:
        """Tokens the row can take beyond `req.cached` with the pages that are free now."""
        lo, hi = 0, req.sequence_len - req.cached
        while lo < hi:                      # largest count with can_reserve true
            mid = (lo + hi + 1) // 2
            if self.cache.can_reserve(req.row, req.cached + mid):
                lo = mid
            else:
                hi = mid - 1
        return lo

    # ------------------------------------------------------------------ after the step
    def sampling_args(self, plan: StepPlan):
        """(temperature, seed, counter) for each entry that samples, in batch order."""
        return [(e.request.sampling.temperature, e.request.sampling.seed, len(e.request.output))
                for e in plan.entries if e.samples]

    def complete(self, plan: StepPlan, tokens: Sequence[int]) -> None:
        """Record a finished step: lengths grow, sampled tokens are appended or end
        their request, finished rows are freed."""
        tokens = list(tokens)
        it = iter(tokens)
        now = time.perf_counter()
        for e in plan.entries:
            req = e.request
            self.cache.commit(req.row, e.start + e.count)
            self.prompt_tokens += max(0, min(e.start + e.count, len(req.ids)) - e.start)
            req.cached = e.start + e.count
            if e.samples:
                self.record(req, int(next(it)), now)
        self.sweep()

    def record(self, req: Request, token: int, now: float) -> None:
        """The stop rule (model/inference_paged.py:200-211): a stop token ends the
        request and is not appended; so does reaching max_new_tokens."""
        if not req.first_token:
            req.first_token = now
        if token in self.stop_ids:
            req.done = True
        else:
            req.output.append(token)
            self.output_tokens += 1
            if req.stream is not None:
                req.stream.put(token)
            if len(req.output) >= req.max_new_tokens:
                req.done = True
        if req.done:
            req.finished = now

    # ------------------------------------------------------------------ invariants
    def check(self) -> None:
        """Rows 0..n_active-1 hold distinct live requests that know their row; the rest
        are empty; the cache agrees (tests call this after every step)."""
        seen = set()
        for i in range(self.max_batch):
            r = self.rows[i]
            if i < self.n_active:
                assert r is not None and r.row == i, f"row {i} is inconsistent"
                assert id(r) not in seen
                seen.add(id(r))
                assert self.cache.active[i]
                assert self.cache.lengths[i] == r.cached
            else:
                assert r is None, f"row {i} beyond the active block holds a request"
                assert not self.cache.active[i]
        self.cache.check()
