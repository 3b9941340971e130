"""The cache manager: pages of keys and values by layer group, block tables, state slots.

What Kapel's `KvCache` does for one page list per sequence shared by all layers
(crates/kapel-models/src/cache.rs:57-72,137-168,751-818) is done here per *group* of layers
with the same needs: layers that see every key form one group, layers with a window of w keys
another, each with pages of its own. After a step that brings a sequence to n positions, a
windowed group gives back every page that lies wholly below n + 1 - w: no later query reads
it (a query that has seen c positions reads from max(0, c - w), crates/kapel-ops/src/paged.rs:65-70).
A block table keeps the logical page -> physical page map of a sequence, with -1 where a page
was given back; kernels never read below the first visible key, so they never meet a hole.

Beside the pages there are slots for per-request state of fixed size (Kapel's `states`,
cache.rs:141-144,846-897): slot 0 belongs to padding rows, a request gets a slot of its own
for its lifetime, and `Plan.fresh` says which slots a step must clear.

The manager is host code only. Device tables are made by an `allocate(shape, dtype)` function
given by the engine, so every decision here can be tested without a GPU.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np

from .pages import CacheFull, PagePool


@dataclass(frozen=True)
class PagedKV:
    """Keys and values of `kv_heads` heads of `head_dim`; `window` None keeps every key."""

    kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed shape (without the slot dimension) in 32-bit floats."""

    shape: Tuple[int, ...]
    dtype: str = "float32"


@dataclass(frozen=True)
class CacheNeeds:
    """What one layer's mixer keeps between steps; both may be None."""

    paged: Optional[PagedKV] = None
    state: Optional[StateSpec] = None


@dataclass
class GroupPlan:
    lines: np.ndarray            # [R] int32: the line (page * page_size + offset) each row writes
    block_table: np.ndarray      # [S, P] int32: logical page -> physical page, -1 for none


@dataclass
class Plan:
    """One step as the kernels see it: rows are the step's tokens, entries its requests."""

    entries: List[Tuple[Hashable, int]]
    positions: np.ndarray        # [R] int32
    row_entry: np.ndarray        # [R] int32: which entry a row belongs to
    row_count: np.ndarray        # [R] int32: positions the row has seen, its own included
    q_start: np.ndarray          # [S] int32: first row of each entry
    q_len: np.ndarray            # [S] int32
    kv_len: np.ndarray           # [S] int32: the entry's length after this step
    slots: np.ndarray            # [S] int32
    fresh: np.ndarray            # [S] bool: the entry's first step (state must start cleared)
    groups: List[GroupPlan]
    taken: List[Tuple[int, Hashable, int, int]] = field(default_factory=list)  # (group, id, logical, physical)
    committed: bool = False

    @property
    def rows(self) -> int:
        return int(self.positions.shape[0])

    @property
    def max_kv_len(self) -> int:
        return int(self.kv_len.max()) if len(self.kv_len) else 0


class PageList:
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
        self.pages: List[PageList] = [PageList() for _ in range(n_groups)]   # -1 where given back
        self.released = [0] * n_groups     # logical pages below this index were given back
        self.slot = slot
        self.fresh = True


class CacheGroup:
    def __init__(self, needs: PagedKV, n_pages: int):
        self.needs = needs
        self.window = needs.window
        self.pool = PagePool(n_pages)
        self.layers: List[int] = []
        self.keys: Dict[int, object] = {}      # layer -> table [pages, kv_heads, page_size, head_dim]
        self.values: Dict[int, object] = {}

    @property
    def name(self) -> str:
        w = "all" if self.window is None else f"window{self.window}"
        return f"{w}/h{self.needs.kv_heads}/d{self.needs.head_dim}"


class CacheManager:
    """Pages by layer group, block tables by sequence, slots by request.

    `needs[layer]` says what the layer that owns cache `layer` keeps. `pages` is the number of
    pages of each group's pool (an int for all, or a dict by `PagedKV`).
    """

    def __init__(
        self,
        needs: Dict[int, CacheNeeds],
        page_size: int,
        pages,
        max_sequences: int,
        allocate: Optional[Callable] = None,
        dtype=None,
    ):
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size = page_size
        self.max_sequences = max_sequences
        self.groups: List[CacheGroup] = []
        self.group_of_layer: Dict[int, int] = {}
        self._by_needs: Dict[PagedKV, int] = {}
        for layer in sorted(needs):
            n = needs[layer]
            if n.paged is None:
                continue
            if n.paged not in self._by_needs:
                count = pages[n.paged] if isinstance(pages, dict) else int(pages)
                self._by_needs[n.paged] = len(self.groups)
                self.groups.append(CacheGroup(n.paged, count))
            g = self._by_needs[n.paged]
            self.groups[g].layers.append(layer)
            self.group_of_layer[layer] = g
        self.state_specs: Dict[int, StateSpec] = {l: n.state for l, n in needs.items() if n.state is not None}
        self.states: Dict[int, object] = {}
        self._sequences: Dict[Hashable, _Sequence] = {}
        self._free_slots = list(range(max_sequences, 0, -1))     # slot 0 is the padding rows'
        self.released_pages = 0
        if allocate is not None:
            self.allocate_tables(allocate, dtype)

    # ------------------------------------------------------------------ device tables
    def allocate_tables(self, allocate: Callable, dtype) -> None:
        """Makes K and V tables [pages, kv_heads, page_size, head_dim] per layer (the keys of one kv
        head in one page lie together, so a kernel fetches them in one piece), and state
        tables [slots + 1, *shape]; they never move afterwards, so a recorded step stays valid."""
        for g in self.groups:
            shape = (max(g.pool.n_pages, 1), g.needs.kv_heads, self.page_size, g.needs.head_dim)
            for layer in g.layers:
                g.keys[layer] = allocate(shape, dtype)
                g.values[layer] = allocate(shape, dtype)
        for layer, spec in self.state_specs.items():
            self.states[layer] = allocate((self.max_sequences + 1, *spec.shape), spec.dtype)

    def tables(self, layer: int):
        g = self.groups[self.group_of_layer[layer]]
        return g.keys[layer], g.values[layer]

    # ------------------------------------------------------------------ sequences
    def __contains__(self, seq_id) -> bool:
        return seq_id in self._sequences

    def sequences(self):
        return list(self._sequences)

    def add_sequence(self, seq_id) -> int:
        if seq_id in self._sequences:
            raise ValueError(f"sequence {seq_id!r} is already in the cache")
        if not self._free_slots:
            raise CacheFull(1, 0, "slots")
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
    def plan(self, entries: Sequence[Tuple[Hashable, int]]) -> Plan:
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
                raise CacheFull(need[g], group.pool.free, group.name)

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
            GroupPlan(np.empty(n_rows, np.int32), np.full((n_entries, max(widest, 1)), -1, np.int32))
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
        return Plan(list(entries), positions, row_entry, row_count, q_start, q_len, kv_len, slots, fresh, group_plans, taken)

    def commit(self, plan: Plan) -> None:
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

    def abort(self, plan: Plan) -> None:
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
