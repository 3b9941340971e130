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
given by the engine, so every decision here can be tested without a GPU. The bookkeeping (free
lists, page lists, the arrays of a step) runs in the host library, `csrc/host/cache_core.cpp`;
this class owns its handle, names the sequences and raises the typed errors.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np

import ctypes

from .pages import CacheFull, host_library


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
    native: object = None        # the manager's own: the entries as the host library takes them
    added: List[Hashable] = field(default_factory=list)   # the step function's: sequences it added for this step

    @property
    def rows(self) -> int:
        return int(self.positions.shape[0])

    @property
    def max_kv_len(self) -> int:
        return int(self.kv_len.max()) if len(self.kv_len) else 0


class CacheGroup:
    def __init__(self, needs: PagedKV, n_pages: int):
        if n_pages < 0:
            raise ValueError(f"a pool cannot have {n_pages} pages")
        self.needs = needs
        self.window = needs.window
        self.n_pages = n_pages
        self.layers: List[int] = []
        self.keys: Dict[int, object] = {}      # layer -> table [pages, kv_heads, page_size, head_dim]
        self.values: Dict[int, object] = {}

    @property
    def name(self) -> str:
        w = "all" if self.window is None else f"window{self.window}"
        return f"{w}/h{self.needs.kv_heads}/d{self.needs.head_dim}"


def _ptr(a: np.ndarray) -> int:
    return a.ctypes.data


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
        self._sequences: Dict[Hashable, int] = {}                # sequence -> its slot (1 ..; 0 is the padding rows')
        self._lib = host_library()
        n_groups = len(self.groups)
        counts = np.asarray([g.n_pages for g in self.groups], np.int32)
        windows = np.asarray([-1 if g.window is None else g.window for g in self.groups], np.int32)
        ip = ctypes.POINTER(ctypes.c_int)
        self._h = self._lib.kc_create(n_groups, page_size, counts.ctypes.data_as(ip), windows.ctypes.data_as(ip), max_sequences)
        if not self._h:
            raise ValueError(f"a cache of {n_groups} groups, pages {counts.tolist()}, {max_sequences} sequences cannot be made")
        self._scratch = np.zeros(max(n_groups, 1), np.int32)
        self._info = np.zeros(7, np.int64)
        self._info_ptr = self._info.ctypes.data
        self._names = 0                                          # counts the sequences that have come or gone
        if allocate is not None:
            self.allocate_tables(allocate, dtype)

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.kc_destroy(self._h)
            self._h = None

    @property
    def released_pages(self) -> int:
        """Pages that windowed groups have given back so far."""
        return int(self._lib.kc_released_pages(self._h))

    # ------------------------------------------------------------------ device tables
    def allocate_tables(self, allocate: Callable, dtype) -> None:
        """Makes K and V tables [pages, kv_heads, page_size, head_dim] per layer (the keys of one kv
        head in one page lie together, so a kernel fetches them in one piece), and state
        tables [slots + 1, *shape]; they never move afterwards, so a recorded step stays valid."""
        for g in self.groups:
            shape = (max(g.n_pages, 1), g.needs.kv_heads, self.page_size, g.needs.head_dim)
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
        slot = self._lib.kc_add(self._h)
        if slot < 1:
            raise CacheFull(1, 0, "slots")
        self._sequences[seq_id] = slot
        self._names += 1
        return slot

    def remove_sequence(self, seq_id) -> None:
        """Gives back everything the sequence holds, last page first."""
        slot = self._sequences.pop(seq_id)
        self._names += 1
        if self._lib.kc_remove(self._h, slot) != 0:
            raise AssertionError(f"sequence {seq_id!r} (slot {slot}) could not give its pages back")

    def length(self, seq_id) -> int:
        return self._lib.kc_length(self._h, self._sequences[seq_id])

    def slot(self, seq_id) -> int:
        return self._sequences[seq_id]

    def free_slots(self) -> int:
        return self._lib.kc_free_slots(self._h)

    def _ints(self, call, *args) -> List[int]:
        r = call(self._h, *args, self._scratch.ctypes.data_as(ctypes.POINTER(ctypes.c_int)))
        if r is not None and r < 0:
            raise KeyError("no such sequence in the cache")
        return self._scratch[: len(self.groups)].tolist()

    def free_pages(self) -> List[int]:
        return self._ints(self._lib.kc_free_pages)

    def total_pages(self) -> List[int]:
        return [g.n_pages for g in self.groups]

    def held_pages(self, seq_id) -> List[int]:
        return self._ints(self._lib.kc_held_pages, self._sequences[seq_id])

    def page_list(self, seq_id, group: int) -> List[int]:
        """The sequence's logical pages in a group, -1 where a page was given back."""
        slot = self._sequences[seq_id]
        n = self._lib.kc_pages_of(self._h, slot, group, None, 0)
        out = np.empty(max(n, 1), np.int32)
        self._lib.kc_pages_of(self._h, slot, group, out.ctypes.data_as(ctypes.POINTER(ctypes.c_int)), n)
        return out[:n].tolist()

    # ------------------------------------------------------------------ arithmetic
    def _pages_for(self, length: int) -> int:
        return -(-length // self.page_size)

    def pages_needed(self, seq_id, count: int) -> List[int]:
        """New pages each group must take for `count` more tokens of `seq_id` (a sequence not
        yet in the cache counts from zero): ceil((len + count) / page) - pages held or passed
        (crates/kapel-models/src/cache.rs:481-486, per group)."""
        return self._ints(self._lib.kc_pages_needed, self._sequences.get(seq_id, 0), int(count))

    def pages_for_tokens(self, tokens: int) -> List[int]:
        """Pages a sequence of `tokens` positions holds at most in each group at one time,
        when it is brought there in one step."""
        return [self._pages_for(tokens) for _ in self.groups]

    def fits(self, entries: Sequence[Tuple[Hashable, int]]) -> bool:
        need = [0] * len(self.groups)
        for seq_id, count in entries:
            for g, n in enumerate(self.pages_needed(seq_id, count)):
                need[g] += n
        return all(n <= f for n, f in zip(need, self.free_pages()))

    # ------------------------------------------------------------------ a step
    def plan(self, entries: Sequence[Tuple[Hashable, int]]) -> Plan:
        """Takes the pages a step needs and describes its rows.

        `entries` is [(sequence, number of new tokens)] in batch order; a sequence appears at
        most once and brings at least one token (crates/kapel-models/src/cache.rs:765-770).
        Raises `CacheFull` and takes nothing if some group lacks pages. Lengths move only at
        `commit`; `abort` gives the pages back.
        """
        entries = list(entries)
        n = len(entries)
        slot_of = self._sequences
        sc = np.empty((2, max(n, 1)), np.int32)                  # slots, counts
        seen = set()
        for e, (seq_id, count) in enumerate(entries):
            if seq_id in seen:
                raise ValueError(f"sequence {seq_id!r} appears twice in one step")
            seen.add(seq_id)
            if count <= 0:
                raise ValueError(f"sequence {seq_id!r} brings no token")
            slot = slot_of.get(seq_id)
            if slot is None:
                raise KeyError(f"sequence {seq_id!r} is not in the cache")
            sc[0, e], sc[1, e] = slot, count
        sc_ptr = sc.ctypes.data
        stride = 4 * sc.shape[1]
        info = self._info
        status = self._lib.kc_plan_prepare(self._h, n, sc_ptr, sc_ptr + stride, self._info_ptr)
        if status == 1:
            raise CacheFull(int(info[5]), int(info[6]), self.groups[int(info[4])].name)
        if status != 0:
            raise AssertionError("the cache's bookkeeping does not know a sequence this manager holds")
        n_rows, widest, n_take = int(info[1]), int(info[2]), int(info[3])
        width = max(widest, 1)
        n_groups = len(self.groups)
        # One buffer for every array of the step: three by row, four by entry, the lines and the
        # block tables of each group, the pages taken, and a byte an entry for `fresh`.
        at_entry = 3 * n_rows
        at_lines = at_entry + 4 * n
        at_tables = at_lines + n_groups * n_rows
        at_taken = at_tables + n_groups * n * width
        at_fresh = at_taken + 4 * n_take
        buf = np.empty(at_fresh + (n + 3) // 4 + 1, np.int32)
        buf[at_tables:at_taken] = -1
        buf[at_fresh:] = 0
        base = buf.ctypes.data
        at = lambda words: base + 4 * words
        line_ptrs = (ctypes.c_void_p * max(n_groups, 1))(*[at(at_lines + g * n_rows) for g in range(n_groups)])
        table_ptrs = (ctypes.c_void_p * max(n_groups, 1))(*[at(at_tables + g * n * width) for g in range(n_groups)])
        got = self._lib.kc_plan_fill(
            self._h, n, sc_ptr, sc_ptr + stride, base, at(n_rows), at(2 * n_rows),
            at(at_entry), at(at_entry + n), at(at_entry + 2 * n), at(at_entry + 3 * n), at(at_fresh),
            ctypes.addressof(line_ptrs), ctypes.addressof(table_ptrs), width, at(at_taken), n_take)
        if got < 0:
            raise AssertionError("the cache's bookkeeping could not take the pages it had counted")
        taken: List[Tuple[int, Hashable, int, int]] = []
        if got:
            name_of = {int(sc[0, e]): entries[e][0] for e in range(n)}
            taken = [(g, name_of[s], logical, page) for g, s, logical, page in buf[at_taken : at_taken + 4 * got].reshape(-1, 4).tolist()]
        group_plans = [
            GroupPlan(buf[at_lines + g * n_rows : at_lines + (g + 1) * n_rows],
                      buf[at_tables + g * n * width : at_tables + (g + 1) * n * width].reshape(n, width))
            for g in range(n_groups)
        ]
        plan = Plan(entries, buf[:n_rows], buf[n_rows : 2 * n_rows], buf[2 * n_rows : 3 * n_rows],
                    buf[at_entry : at_entry + n], buf[at_entry + n : at_entry + 2 * n], buf[at_entry + 2 * n : at_entry + 3 * n],
                    buf[at_entry + 3 * n : at_entry + 4 * n], buf[at_fresh:].view(np.bool_)[:n], group_plans, taken)
        plan.native = (self._names, sc, n)
        return plan

    def _entries_arrays(self, entries):
        live = [(self._sequences[s], c) for s, c in entries]
        arr = np.asarray(live, np.int32).reshape(-1, 2)
        return np.ascontiguousarray(arr[:, 0]), np.ascontiguousarray(arr[:, 1])

    def commit(self, plan: Plan) -> None:
        """The step's kernels are enqueued: lengths advance, and windowed groups give back the
        pages no later query can read."""
        if plan.committed:
            raise ValueError("a plan is committed once")
        plan.committed = True
        native = plan.native
        if native is not None and native[0] == self._names:       # no sequence has come or gone since the plan
            sc, n = native[1], native[2]
            ptr = sc.ctypes.data
            r = self._lib.kc_commit(self._h, n, ptr, ptr + 4 * sc.shape[1])
        else:
            slots, counts = self._entries_arrays(plan.entries)
            r = self._lib.kc_commit(self._h, len(plan.entries), _ptr(slots), _ptr(counts))
        if r < 0:
            raise AssertionError("a committed plan names a sequence the cache does not hold")

    def abort(self, plan: Plan) -> None:
        """The step did not run: the pages it took go back, newest first."""
        if plan.committed:
            raise ValueError("a committed plan cannot be aborted")
        quads = [(g, self._sequences[s], logical, page) for g, s, logical, page in plan.taken if s in self._sequences]
        if quads:
            raw = np.asarray(quads, np.int32)
            self._lib.kc_abort(self._h, len(quads), _ptr(raw))
        plan.taken.clear()
        plan.committed = True

    # ------------------------------------------------------------------ checks
    def check(self) -> None:
        """No page lost, none held twice: every held page belongs to exactly one sequence."""
        msg = ctypes.create_string_buffer(512)
        if self._lib.kc_check(self._h, msg, 512):
            raise AssertionError(msg.value.decode())
        slots = list(self._sequences.values())
        if len(set(slots)) != len(slots) or 0 in slots:
            raise AssertionError("a slot is held twice or is the padding slot")
        if len(slots) + self.free_slots() != self.max_sequences:
            raise AssertionError("a slot was lost")
