"""The cache manager: paged keys and values, block tables, and fixed-size state slots.

What the reference has (model/qwen/qwen_kv_paged.py:34-127): per-layer K and V pools
`[num_blocks+1, Hkv, BS, D]` with page 0 as the null page, one int32 block table for
all layers, host-side lengths, and assign / release / move_row.  What is added here:

* **Groups.**  Layers whose mixers ask for the same page shape and the same window
  share one group: one allocator, one block table, one pool tensor with a leading
  axis over the group's layers.  A model whose layers differ (all keys in some, a
  window of keys in others) gets one group for each need, each with pages of its own.
* **Lazy pages.**  `reserve(row, new_len)` takes pages only for the slots about to be
  written (the reference reserves the worst case at admission,
  model/inference_paged.py:150-157).  It either takes every page it needs in every
  group or changes nothing.
* **Windows give pages back.**  `commit(row, new_len)` frees the pages of a windowed
  group that no later query can see.
* **State slots.**  A mixer may ask for a fixed-size tensor per request; it lives at
  the request's row in `[max_rows, *shape]`, is zeroed on `assign`, and moves with
  `move_row`.

Everything a scheduler decides (which pages a row owns, how long it is) lives on the
host; `flush()` copies the table rows that changed to the device between steps.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .allocator import OutOfPages, PageAllocator, pages_for


@dataclass(frozen=True)
class PagedKVSpec:
    """Keys and values of `num_kv_heads` heads of `head_dim`; `window` keys are kept
    (None: all of them)."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateSpec:
    """A tensor of fixed shape per request."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass(frozen=True)
class CacheNeeds:
    """What one run of a layer asks of the cache manager."""
    paged: Optional[PagedKVSpec] = None
    state: Optional[StateSpec] = None


class PageGroup:
    """Pages, allocator and block table of the layer runs that share one PagedKVSpec."""

    def __init__(self, spec: PagedKVSpec, entries: List[int], max_rows: int, table_width: int,
                 page_size: int, num_pages: int, dtype: torch.dtype, device):
        self.spec = spec
        self.entries = entries
        self.page_size = page_size
        self.allocator = PageAllocator(num_pages)
        shape = (len(entries), num_pages + 1, spec.num_kv_heads, page_size, spec.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        self.table = torch.zeros((max_rows, table_width), dtype=torch.int32, device=device)
        self.host_table = torch.zeros((max_rows, table_width), dtype=torch.int32)
        # Logical block -> page for each row; 0 where nothing is held (never written,
        # or given back after the window passed).
        self.row_pages: List[List[int]] = [[] for _ in range(max_rows)]
        self.freed_upto: List[int] = [0] * max_rows     # blocks below this were given back (window)
        self.dirty: set[int] = set()

    def slot_of(self, entry: int) -> int:
        return self.entries.index(entry)

    def first_needed_block(self, next_pos: int) -> int:
        """The lowest logical block that a query at `next_pos` or later can still see."""
        if self.spec.window is None:
            return 0
        return max(0, next_pos - self.spec.window + 1) // self.page_size

    def owned(self, row: int) -> List[int]:
        return [p for p in self.row_pages[row] if p != 0]


class CacheManager:
    def __init__(self, needs: Sequence[Optional[CacheNeeds]], max_rows: int, max_len: int,
                 page_size: int, num_pages: int, dtype: torch.dtype, device="cuda"):
        """`needs[i]` is what order entry i asks for (None: nothing of its own)."""
        self.max_rows, self.max_len, self.page_size = max_rows, max_len, page_size
        self.table_width = pages_for(max_len, page_size)
        self.device = torch.device(device)
        self.dtype = dtype
        self.lengths: List[int] = [0] * max_rows
        self.active: List[bool] = [False] * max_rows

        by_spec: Dict[PagedKVSpec, List[int]] = {}
        for i, n in enumerate(needs):
            if n is not None and n.paged is not None:
                by_spec.setdefault(n.paged, []).append(i)
        self.groups: List[PageGroup] = [
            PageGroup(spec, entries, max_rows, self.table_width, page_size, num_pages, dtype, self.device)
            for spec, entries in by_spec.items()]
        self.group_of_entry: Dict[int, int] = {
            e: gi for gi, g in enumerate(self.groups) for e in g.entries}

        self.states: Dict[int, torch.Tensor] = {}
        for i, n in enumerate(needs):
            if n is not None and n.state is not None:
                self.states[i] = torch.zeros((max_rows, *n.state.shape), dtype=n.state.dtype,
                                             device=self.device)
        self._staging: List[Tuple[torch.Tensor, Optional[torch.cuda.Event]]] = []
        self._staging_next = 0

    @staticmethod
    def bytes_per_page(needs: Sequence[Optional[CacheNeeds]], page_size: int, dtype: torch.dtype) -> int:
        """Device bytes that one more page per group costs (keys and values of every layer run
        of every group), for sizing the pool from a memory budget."""
        item = torch.empty((), dtype=dtype).element_size()
        return sum(2 * n.paged.num_kv_heads * page_size * n.paged.head_dim * item
                   for n in needs if n is not None and n.paged is not None)

    # ------------------------------------------------------------------ views for mixers
    def pools(self, entry: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """K and V pools `[pages+1, Hkv, BS, D]` of one order entry."""
        g = self.groups[self.group_of_entry[entry]]
        s = g.slot_of(entry)
        return g.k[s], g.v[s]

    def block_table(self, entry: int) -> torch.Tensor:
        """Device block table `[max_rows, W]` of the group that `entry` belongs to."""
        return self.groups[self.group_of_entry[entry]].table

    def window(self, entry: int) -> Optional[int]:
        return self.groups[self.group_of_entry[entry]].spec.window

    def state(self, entry: int) -> torch.Tensor:
        """State slots `[max_rows, *shape]` of one order entry."""
        return self.states[entry]

    # ------------------------------------------------------------------ rows
    def assign(self, row: int) -> None:
        """Open an empty row for a new request: length 0, no pages, state zeroed."""
        if self.active[row]:
            raise ValueError(f"row {row} is still in use")
        self.active[row] = True
        self.lengths[row] = 0
        for t in self.states.values():
            t[row].zero_()

    def pages_needed(self, row: int, new_len: int) -> List[int]:
        """Pages each group still lacks for the row to hold `new_len` tokens.

        A row's pages are taken in order and given back only from the front (behind a
        window), so the blocks it lacks are exactly those past the end of its list, from
        the first block a later query can still see.
        """
        last = pages_for(new_len, self.page_size)              # exclusive
        out = []
        for g in self.groups:
            first = g.first_needed_block(self.lengths[row])
            out.append(max(0, last - max(first, len(g.row_pages[row]))))
        return out

    def can_reserve(self, row: int, new_len: int) -> bool:
        if new_len > self.max_len:
            return False
        return all(n <= g.allocator.n_free for n, g in zip(self.pages_needed(row, new_len), self.groups))

    def reserve(self, row: int, new_len: int) -> bool:
        """Take the pages the row needs to grow to `new_len` tokens, in every group.

        Returns False and changes nothing if any group has too few free pages.
        Raises if `new_len` exceeds the row's table.
        """
        if not self.active[row]:
            raise ValueError(f"row {row} is not in use")
        if new_len > self.max_len:
            raise ValueError(f"{new_len} tokens exceed the row limit of {self.max_len}")
        needs = self.pages_needed(row, new_len)
        if any(n > g.allocator.n_free for n, g in zip(needs, self.groups)):
            return False
        last = pages_for(new_len, self.page_size)
        for g, need in zip(self.groups, needs):
            if need == 0:
                continue
            have = g.row_pages[row]
            first = g.first_needed_block(self.lengths[row])
            while len(have) < min(first, last):                 # blocks no query will see again
                have.append(0)
            pages = g.allocator.alloc(need)
            start = len(have)
            have.extend(pages)
            g.host_table[row, start:start + need] = torch.tensor(pages, dtype=torch.int32)
            g.dirty.add(row)
        return True

    def commit(self, row: int, new_len: int) -> None:
        """The row now holds `new_len` tokens; pages behind every window go back."""
        if new_len < self.lengths[row]:
            raise ValueError("a row does not shrink")
        self.lengths[row] = new_len
        for g in self.groups:
            if g.spec.window is None:
                continue
            keep_from = g.first_needed_block(new_len)
            have = g.row_pages[row]
            upto = min(keep_from, len(have))
            gone = [b for b in range(g.freed_upto[row], upto) if have[b] != 0]
            g.freed_upto[row] = max(g.freed_upto[row], upto)
            if gone:
                g.allocator.free([have[b] for b in gone])
                for b in gone:
                    have[b] = 0
                    g.host_table[row, b] = 0
                g.dirty.add(row)

    def release(self, row: int) -> None:
        """Close a row: every page it holds goes back, its table row points at the null page."""
        if not self.active[row]:
            raise ValueError(f"row {row} is not in use")
        for g in self.groups:
            owned = g.owned(row)
            if owned:
                g.allocator.free(owned)
            if g.row_pages[row]:
                g.host_table[row].zero_()
                g.dirty.add(row)
            g.row_pages[row] = []
            g.freed_upto[row] = 0
        self.lengths[row] = 0
        self.active[row] = False

    def move_row(self, src: int, dst: int) -> None:
        """Relocate a live row; only its table row and state slot move, never the pages
        (model/qwen/qwen_kv_paged.py:102-109)."""
        if src == dst:
            return
        if not self.active[src]:
            raise ValueError(f"row {src} is not in use")
        if self.active[dst]:
            raise ValueError(f"row {dst} is still in use; release it first")
        for g in self.groups:
            g.row_pages[dst], g.row_pages[src] = g.row_pages[src], []
            g.freed_upto[dst], g.freed_upto[src] = g.freed_upto[src], 0
            g.host_table[dst].copy_(g.host_table[src])
            g.host_table[src].zero_()
            g.dirty.update((src, dst))
        for t in self.states.values():
            t[dst].copy_(t[src])
        self.lengths[dst], self.lengths[src] = self.lengths[src], 0
        self.active[dst], self.active[src] = True, False

    # ------------------------------------------------------------------ device tables
    def _stage(self, n_rows: int) -> torch.Tensor:
        """A pinned buffer that no copy still in flight reads from."""
        if self.device.type != "cuda":
            return torch.empty((n_rows, self.table_width), dtype=torch.int32)
        if not self._staging:
            for _ in range(4):
                buf = torch.empty((self.max_rows * max(1, len(self.groups)), self.table_width),
                                  dtype=torch.int32).pin_memory()
                self._staging.append([buf, None])
        slot = self._staging[self._staging_next]
        self._staging_next = (self._staging_next + 1) % len(self._staging)
        if slot[1] is not None:
            slot[1].synchronize()
        return slot[0]

    def flush(self) -> None:
        """Copy the table rows that changed since the last flush to the device, on the
        current stream.  Call between steps, before the step that uses them."""
        total = sum(len(g.dirty) for g in self.groups)
        if total == 0:
            return
        stage = self._stage(total)
        i = 0
        for g in self.groups:
            for row in sorted(g.dirty):
                stage[i].copy_(g.host_table[row])
                g.table[row].copy_(stage[i], non_blocking=True)
                i += 1
            g.dirty.clear()
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record()
            self._staging[(self._staging_next - 1) % len(self._staging)][1] = ev

    # ------------------------------------------------------------------ accounting
    def free_pages(self) -> List[int]:
        return [g.allocator.n_free for g in self.groups]

    def bytes_per_token(self) -> int:
        item = torch.empty((), dtype=self.dtype).element_size()
        return sum(2 * len(g.entries) * g.spec.num_kv_heads * g.spec.head_dim * item for g in self.groups)

    def check(self) -> None:
        """No page lost, held twice or freed twice; tables agree with ownership."""
        for g in self.groups:
            g.allocator.check()
            owned: List[int] = []
            for row in range(self.max_rows):
                pages = g.owned(row)
                if pages and not self.active[row]:
                    raise AssertionError(f"inactive row {row} owns pages")
                owned += pages
                have = g.row_pages[row]
                for b in range(self.table_width):
                    want = have[b] if b < len(have) else 0
                    if int(g.host_table[row, b]) != want:
                        raise AssertionError(f"table of row {row} block {b} disagrees with ownership")
            if len(owned) != len(set(owned)):
                raise AssertionError("a page is held by two rows")
            if len(owned) != g.allocator.n_used or not all(g.allocator.holds(p) for p in owned):
                raise AssertionError("pages owned by rows differ from pages marked used")
            if PageAllocator.NULL in owned:
                raise AssertionError("the null page is owned")
