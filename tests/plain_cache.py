"""A plain cache manager for the tests: pools of pages by layer group, page lists by sequence, state
slots and the arrays of a step, in Python lists and numpy, sharing no code with the package.

The package does this bookkeeping in a small C++ library; the tests drive both with the same
random requests and want the same pages, the same arrays and the same free lists from both. The
arithmetic follows Kapel's `KvCache` (crates/kapel-models/src/cache.rs:419-433 free list,
:481-486 pages needed, :751-818 the plan of a pass), per group of layers, plus the window's
release: after a step that brings a sequence to n positions, a group with a window of w keys gives
back every page wholly below n + 1 - w (a query that has seen c positions reads from
max(0, c - w), crates/kapel-ops/src/paged.rs:65-70).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np


@dataclass(frozen=True)
class PlainKV:
    kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass
class PlainGroupPlan:
    lines: np.ndarray
    block_table: np.ndarray


@dataclass
class PlainPlan:
    entries: List[Tuple[Hashable, int]]
    positions: np.ndarray
    row_entry: np.ndarray
    row_count: np.ndarray
    q_start: np.ndarray
    q_len: np.ndarray
    kv_len: np.ndarray
    slots: np.ndarray
    fresh: np.ndarray
    groups: List[PlainGroupPlan]
    taken: List[Tuple[int, Hashable, int, int]] = field(default_factory=list)
    committed: bool = False

    @property
    def rows(self) -> int:
        return int(self.positions.shape[0])


class PlainCacheFull(RuntimeError):
    """A pool has fewer free pages than a step needs."""

    def __init__(self, needed: int, free: int, group: str = ""):
        self.needed, self.free, self.group = needed, free, group
        where = f" in group {group}" if group else ""
        super().__init__(f"cache full{where}: {needed} pages needed, {free} free")


class PlainPagePool:
    """`n_pages` pages numbered from 0; the page freed last is taken first."""

    def __init__(self, n_pages: int):
        if n_pages < 0:
            raise ValueError(f"a pool cannot have {n_pages} pages")
        self.n_pages = n_pages
        # Pop takes from the end: page 0 first in a fresh pool.
        self._free: List[int] = list(range(n_pages - 1, -1, -1))
        self._held = [False] * n_pages

    @property
    def free(self) -> int:
        return len(self._free)

    @property
    def held(self) -> int:
        return self.n_pages - len(self._free)

    def take(self) -> int:
        if not self._free:
            raise PlainCacheFull(1, 0)
        page = self._free.pop()
        if self._held[page]:
            raise AssertionError(f"page {page} was on the free list while held")
        self._held[page] = True
        return page

    def give(self, page: int) -> None:
        if not 0 <= page < self.n_pages:
            raise ValueError(f"page {page} is not of this pool (0..{self.n_pages - 1})")
        if not self._held[page]:
            raise ValueError(f"page {page} is given back twice")
        self._held[page] = False
        self._free.append(page)

    def is_held(self, page: int) -> bool:
        return self._held[page]

    def check(self) -> None:
        """Every page is free or held, never both, none lost."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise AssertionError("a page is on the free list twice")
        for p in range(self.n_pages):
            if self._held[p] == (p in free):
                raise AssertionError(f"page {p}: held={self._held[p]} but on the free list={p in free}")


class PlainPageList:
    """A sequence's logical pages in one group, as a list that is also an int32 array: a step's
    block-table row is a slice of it, not a conversion of a Python list every step."""

    __slots__ = ("a", "n")

    def __init__(self):
        self.a = np.empty(16, np.int32)
        self.n = 0

    def __len__(self) -> int:
        return self.n

    def __iter__(self):
        return iter(self.a[: self.n].tolist())

    def __reversed__(self):
        return iter(self.a[: self.n][::-1].tolist())

    def __getitem__(self, i: int) -> int:
        if not -self.n <= i < self.n:
            raise IndexError(i)
        return int(self.a[i if i >= 0 else self.n + i])

    def __setitem__(self, i: int, page: int) -> None:
        if not 0 <= i < self.n:
            raise IndexError(i)
        self.a[i] = page

    def append(self, page: int) -> None:
        if self.n == self.a.size:
            self.a = np.concatenate([self.a, np.empty(self.a.size, np.int32)])
        self.a[self.n] = page
        self.n += 1

    def pop(self) -> int:
        if self.n == 0:
            raise IndexError("pop from no pages")
        self.n -= 1
        return int(self.a[self.n])

    def array(self) -> np.ndarray:
        return self.a[: self.n]


class _Sequence:
    __slots__ = ("length", "pages", "released", "slot", "fresh")

    def __init__(self, n_groups: int, slot: int):
        self.length = 0
        self.pages: List[PlainPageList] = [PlainPageList() for _ in range(n_groups)]   # -1 where given back
        self.released = [0] * n_groups     # logical pages below this index were given back
        self.slot = slot
        self.fresh = True


class PlainCacheGroup:
    def __init__(self, window: Optional[int], n_pages: int):
        self.window = window
        self.pool = PlainPagePool(n_pages)

    @property
    def name(self) -> str:
        return "all" if self.window is None else f"window{self.window}"


class PlainCacheManager:
    """`groups` is [(window or None, pages of the pool)], one entry a group of layers."""

    def __init__(self, groups: Sequence[Tuple[Optional[int], int]], page_size: int, max_sequences: int):
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size = page_size
        self.max_sequences = max_sequences
        self.groups: List[PlainCacheGroup] = [PlainCacheGroup(w, n) for w, n in groups]
        self._sequences: Dict[Hashable, _Sequence] = {}
        self._free_slots = list(range(max_sequences, 0, -1))     # slot 0 is the padding rows'
        self.released_pages = 0

    # ------------------------------------------------------------------ sequences
    def __contains__(self, seq_id) -> bool:
        return seq_id in self._sequences

    def sequences(self):
        return list(self._sequences)

    def add_sequence(self, seq_id) -> int:
        if seq_id in self._sequences:
            raise ValueError(f"sequence {seq_id!r} is already in the cache")
        if not self._free_slots:
            raise PlainCacheFull(1, 0, "slots")
        slot = self._free_slots.pop()
        self._sequences[seq_id] = _Sequence(len(self.groups), slot)
        return slot

    def remove_sequence(self, seq_id) -> None:
        """Gives back everything the sequence holds, last page first."""
        seq = self._sequences.pop(seq_id)
        for g, group in enumerate(self.groups):
            for page in reversed(seq.pages[g]):
                if page >= 0:
                    group.pool.give(page)
        self._free_slots.append(seq.slot)

    def length(self, seq_id) -> int:
        return self._sequences[seq_id].length

    def slot(self, seq_id) -> int:
        return self._sequences[seq_id].slot

    def free_slots(self) -> int:
        return len(self._free_slots)

    def free_pages(self) -> List[int]:
        return [g.pool.free for g in self.groups]

    def total_pages(self) -> List[int]:
        return [g.pool.n_pages for g in self.groups]

    def held_pages(self, seq_id) -> List[int]:
        seq = self._sequences[seq_id]
        return [sum(1 for p in seq.pages[g] if p >= 0) for g in range(len(self.groups))]

    # ------------------------------------------------------------------ arithmetic
    def _pages_for(self, length: int) -> int:
        return -(-length // self.page_size)

    def pages_needed(self, seq_id, count: int) -> List[int]:
        """New pages each group must take for `count` more tokens of `seq_id` (a sequence not
        yet in the cache counts from zero): ceil((len + count) / page) - pages held or passed
        (crates/kapel-models/src/cache.rs:481-486, per group)."""
        seq = self._sequences.get(seq_id)
        length = seq.length if seq is not None else 0
        have = [len(seq.pages[g]) if seq is not None else 0 for g in range(len(self.groups))]
        return [self._pages_for(length + count) - have[g] for g in range(len(self.groups))]

    def pages_for_tokens(self, tokens: int) -> List[int]:
        """Pages a sequence of `tokens` positions holds at most in each group at one time,
        when it is brought there in one step."""
        return [self._pages_for(tokens) for _ in self.groups]

    def fits(self, entries: Sequence[Tuple[Hashable, int]]) -> bool:
        need = [0] * len(self.groups)
        for seq_id, count in entries:
            for g, n in enumerate(self.pages_needed(seq_id, count)):
                need[g] += n
        return all(n <= g.pool.free for n, g in zip(need, self.groups))

    # ------------------------------------------------------------------ a step
    def plan(self, entries: Sequence[Tuple[Hashable, int]]) -> "PlainPlan":
        """Takes the pages a step needs and describes its rows.

        `entries` is [(sequence, number of new tokens)] in batch order; a sequence appears at
        most once and brings at least one token (crates/kapel-models/src/cache.rs:765-770).
        Raises `CacheFull` and takes nothing if some group lacks pages. Lengths move only at
        `commit`; `abort` gives the pages back.
        """
        seen = set()
        for seq_id, count in entries:
            if seq_id in seen:
                raise ValueError(f"sequence {seq_id!r} appears twice in one step")
            seen.add(seq_id)
            if count <= 0:
                raise ValueError(f"sequence {seq_id!r} brings no token")
            if seq_id not in self._sequences:
                raise KeyError(f"sequence {seq_id!r} is not in the cache")
        need = [0] * len(self.groups)
        for seq_id, count in entries:
            for g, n in enumerate(self.pages_needed(seq_id, count)):
                need[g] += n
        for g, group in enumerate(self.groups):
            if need[g] > group.pool.free:
                raise PlainCacheFull(need[g], group.pool.free, group.name)

        ps = self.page_size
        n_rows = sum(c for _, c in entries)
        n_entries = len(entries)
        positions = np.empty(n_rows, np.int32)
        row_entry = np.empty(n_rows, np.int32)
        row_count = np.empty(n_rows, np.int32)
        q_start = np.empty(n_entries, np.int32)
        q_len = np.empty(n_entries, np.int32)
        kv_len = np.empty(n_entries, np.int32)
        slots = np.empty(n_entries, np.int32)
        fresh = np.zeros(n_entries, bool)
        widest = max((self._pages_for(self._sequences[s].length + c) for s, c in entries), default=0)
        group_plans = [
            PlainGroupPlan(np.empty(n_rows, np.int32), np.full((n_entries, max(widest, 1)), -1, np.int32))
            for _ in self.groups
        ]
        taken: List[Tuple[int, Hashable, int, int]] = []
        r = 0
        for e, (seq_id, count) in enumerate(entries):
            seq = self._sequences[seq_id]
            start, end = seq.length, seq.length + count
            q_start[e], q_len[e], kv_len[e] = r, count, end
            slots[e], fresh[e] = seq.slot, seq.fresh
            if count == 1:
                positions[r], row_entry[r], row_count[r] = start, e, end
            else:
                positions[r : r + count] = np.arange(start, end, dtype=np.int32)
                row_entry[r : r + count] = e
                row_count[r : r + count] = np.arange(start + 1, end + 1, dtype=np.int32)
            for g, group in enumerate(self.groups):
                pages = seq.pages[g]
                while len(pages) < self._pages_for(end):
                    page = group.pool.take()
                    taken.append((g, seq_id, len(pages), page))
                    pages.append(page)
                table = pages.array()
                group_plans[g].block_table[e, : len(pages)] = table
                if count == 1:                                   # a decoded token: no arrays to build
                    group_plans[g].lines[r] = int(table[start // ps]) * ps + start % ps
                else:
                    pos = positions[r : r + count]
                    group_plans[g].lines[r : r + count] = table[pos // ps] * ps + pos % ps
            r += count
        return PlainPlan(list(entries), positions, row_entry, row_count, q_start, q_len, kv_len, slots, fresh, group_plans, taken)

    def commit(self, plan: "PlainPlan") -> None:
        """The step's kernels are enqueued: lengths advance, and windowed groups give back the
        pages no later query can read."""
        if plan.committed:
            raise ValueError("a plan is committed once")
        plan.committed = True
        for seq_id, count in plan.entries:
            seq = self._sequences[seq_id]
            seq.length += count
            seq.fresh = False
            for g, group in enumerate(self.groups):
                if group.window is None:
                    continue
                # The next query has seen at least length + 1 positions and reads from
                # (length + 1) - window on; pages wholly below that are done.
                first_needed = seq.length + 1 - group.window
                if first_needed <= 0:
                    continue
                upto = min(first_needed // self.page_size, len(seq.pages[g]))
                for p in range(seq.released[g], upto):
                    if seq.pages[g][p] >= 0:
                        group.pool.give(seq.pages[g][p])
                        seq.pages[g][p] = -1
                        self.released_pages += 1
                seq.released[g] = max(seq.released[g], upto)

    def abort(self, plan: "PlainPlan") -> None:
        """The step did not run: the pages it took go back, newest first."""
        if plan.committed:
            raise ValueError("a committed plan cannot be aborted")
        for g, seq_id, logical, page in reversed(plan.taken):
            seq = self._sequences.get(seq_id)
            if seq is not None and len(seq.pages[g]) == logical + 1 and seq.pages[g][logical] == page:
                seq.pages[g].pop()
                self.groups[g].pool.give(page)
        plan.taken.clear()
        plan.committed = True

    # ------------------------------------------------------------------ checks
    def check(self) -> None:
        """No page lost, none held twice: every held page belongs to exactly one sequence."""
        for g, group in enumerate(self.groups):
            group.pool.check()
            owners: Dict[int, Hashable] = {}
            for seq_id, seq in self._sequences.items():
                for page in seq.pages[g]:
                    if page < 0:
                        continue
                    if page in owners:
                        raise AssertionError(f"group {group.name}: page {page} held by {owners[page]!r} and {seq_id!r}")
                    if not group.pool.is_held(page):
                        raise AssertionError(f"group {group.name}: page {page} of {seq_id!r} is on the free list")
                    owners[page] = seq_id
            if len(owners) != group.pool.held:
                raise AssertionError(
                    f"group {group.name}: {group.pool.held} pages held, {len(owners)} owned: pages lost"
                )
        slots = [s.slot for s in self._sequences.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots) or 0 in slots:
            raise AssertionError("a slot is held twice, is free while held, or is the padding slot")
        if len(slots) + len(self._free_slots) != self.max_sequences:
            raise AssertionError("a slot was lost")
