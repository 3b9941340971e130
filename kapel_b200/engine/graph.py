"""Decode steps recorded once as CUDA graphs and replayed.

A pass in which every request brings one token has the same kernels at the same sizes as any
other such pass of as many rows, so it is captured once per (rows, block-table width) bucket
and replayed with new inputs copied into the same buffers: one host-to-device copy and one
graph launch instead of a few hundred kernel launches. Kapel does the same with its
`record_step` / `replay_step` (crates/kapel-models/src/model.rs:1055-1255) and the row buckets of
its engine (crates/kapel-infer/src/engine.rs:166-177). Padding rows have seen nothing and write
nowhere (count 0, line -1), so they need no scratch pages. The cache tables never move, so a
recording stays valid for the engine's life.
"""
from __future__ import annotations

import dataclasses
import gc
import weakref
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from .batch import GroupBatch, StepBatch, decode_split, sm_count

ROW_BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256)
WIDTH_STEP = 64          # block-table widths are rounded up to a multiple of this many pages


class StaticBatch:
    """A batch of fixed size whose inputs live in one device buffer that replays rewrite."""

    def __init__(self, rows: int, width: int, n_groups: int, device, chunk: int, page_size: int):
        self.rows = self.entries = rows
        self.width = width
        self.chunk = chunk
        self.memo: Dict[object, object] = {}
        sizes = [rows] * 6 + [rows, rows * width] * n_groups
        self.total = sum(sizes)
        # Two pinned staging buffers taken in turn: the next pass can be written while the copy of
        # the last one may still be in flight. Each has an event recorded behind its copy; the host
        # waits for it before it writes that buffer again, so a caller that enqueues pass after
        # pass without synchronising is held back once it is two passes ahead of the device and
        # never rewrites inputs that a copy has yet to read.
        self.hosts = [torch.empty((self.total,), dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self.copied = [torch.cuda.Event() for _ in range(2)]
        self.in_flight = [False, False]
        self.turn = 0
        self.dev = torch.empty((self.total,), dtype=torch.int32, device=device)
        views, at = [], 0
        for n in sizes:
            views.append(self.dev[at : at + n])
            at += n
        self.ids, self.positions, self.row_entry, self.row_count, self.want_rows, self.slots = views[:6]
        self.groups = [GroupBatch(views[6 + 2 * g], views[7 + 2 * g].view(rows, width)) for g in range(n_groups)]
        self._sizes = sizes
        self.fixed_slots = max(1, -(-(width * page_size) // chunk))
        # the tensor-core attention kernel's tiles: every row a tile of one token
        every = torch.arange(rows, dtype=torch.int32, device=device)
        self._tiles = (every, every.clone(), torch.ones(rows, dtype=torch.int32, device=device))
        self._longest = width * page_size
        self._device = device
        self._mma = {}
        self.h2d_bytes = self.total * 4

    def attention_slots(self, window: Optional[int]) -> int:
        n = self.fixed_slots
        if window:
            n = min(n, (window - 1) // self.chunk + 2)
        return max(1, n)

    def attention_tiles(self, heads_per_kv: int, kv_heads: int, window: Optional[int] = None, head_dim: int = 256,
                        prompt_kernel: str = "mma"):
        if (kv_heads, window) not in self._mma:
            self._mma[(kv_heads, window)] = decode_split(self.rows * kv_heads, self._longest, sm_count(self._device), window, True)
        split, slots = self._mma[(kv_heads, window)]
        return heads_per_kv, self._tiles, split, slots, True  # one token a row: heads_per_kv rows a tile, slots from its window's start

    def fill(self, plan, ids) -> None:
        """Writes a plan of at most `rows` single-token entries into the buffers; the rest are
        padding rows."""
        which = self.fill_host(plan)
        self.set_ids(which, ids, plan.rows)
        self.upload(which)

    def set_ids(self, which: int, ids, n: int) -> None:
        flat = self.hosts[which].numpy()
        flat[:n] = np.asarray(ids, np.int32)
        flat[n : self.rows] = 0

    def upload(self, which: int) -> None:
        """One copy of everything a pass reads; the other staging buffer takes the next pass."""
        self.dev.copy_(self.hosts[which], non_blocking=True)
        self.copied[which].record()
        self.in_flight[which] = True
        self.turn = which ^ 1

    def fill_host(self, plan) -> int:
        """Everything of a plan but its token ids into the staging buffer whose turn it is; returns
        which. Nothing is copied to the device yet."""
        n = plan.rows
        rows, width = self.rows, self.width
        which = self.turn
        if self.in_flight[which]:
            self.copied[which].synchronize()                 # the copy that last read this buffer is done
            self.in_flight[which] = False
        flat = self.hosts[which].numpy()
        at = rows                                            # the ids come first

        def put(values, pad):
            nonlocal at
            flat[at : at + n] = values
            flat[at + n : at + rows] = pad
            at += rows

        put(plan.positions, 0)
        put(plan.row_entry, 0)
        flat[at - rows + n : at] = np.arange(n, rows, dtype=np.int32)     # a padding row is its own entry
        put(plan.row_count, 0)
        put(np.arange(n, dtype=np.int32), 0)
        flat[at - rows + n : at] = np.arange(n, rows, dtype=np.int32)     # every row is wanted
        put(plan.slots, 0)
        for g in plan.groups:
            put(g.lines, -1)
            table = flat[at : at + rows * width].reshape(rows, width)
            table[:] = -1
            w = g.block_table.shape[1]
            table[:n, :w] = g.block_table
            at += rows * width
        return which


RETRY_AFTER = 256        # passes before a size that could not be recorded is tried again (crates/kapel-infer/src/engine.rs:521-526)


class CaptureFailed(RuntimeError):
    """A decode pass could not be recorded; the pass itself is not lost (it runs eagerly)."""


class DecodeGraphs:
    def __init__(self, engine, max_rows: int):
        # A weak reference: an engine and its recordings must not form a cycle, or an engine that
        # is no longer used would be destroyed by the cyclic collector at a time of its choosing,
        # and destroying a recording while another engine is capturing one invalidates the capture.
        self._engine = weakref.ref(engine)
        self.max_rows = max_rows
        self.graphs: Dict[Tuple[int, int], Tuple[torch.cuda.CUDAGraph, StaticBatch, torch.Tensor]] = {}
        self.replays = 0
        self.replayed_kernels = 0      # kernels that ran inside replays (the library counts only launches it makes itself)
        self.pool = None
        self.passes = 0                # decode passes offered to `run`, recorded or not
        self.unrecordable: Dict[Tuple[int, int], int] = {}     # bucket -> the pass at which its recording failed
        self.failed_captures = 0
        self.last_capture_error: Optional[str] = None
        # Failure injection on the host, for tests: this many of the next recordings raise inside the capture.
        self.fail_next_captures = 0

    def bucket(self, rows: int, width: int) -> Optional[Tuple[int, int]]:
        for b in ROW_BUCKETS:
            if b >= rows:
                return b, -(-width // WIDTH_STEP) * WIDTH_STEP
        return None

    def prepare(self, plan):
        """Stages a decode-only plan whose token ids are not known yet: (plan, bucket, staging
        buffer), or None if its bucket has no recording so far."""
        width = max(g.block_table.shape[1] for g in plan.groups) if plan.groups else 1
        key = self.bucket(plan.rows, width)
        if key is None or key not in self.graphs:
            return None
        return plan, key, self.graphs[key][1].fill_host(plan)

    def run_prepared(self, prepared, ids=None, ids_device=None) -> torch.Tensor:
        """The staged pass with its token ids: one copy, one replay. The ids come from the host
        (`ids`) or are already on the device (`ids_device`, int32, one a row in the staged order:
        what the sampling kernel of the pass before wrote), in which case nothing waits for them."""
        plan, key, which = prepared
        graph, static, out = self.graphs[key]
        if ids_device is None:
            static.set_ids(which, ids, plan.rows)
        static.upload(which)
        if ids_device is not None:
            static.ids[: plan.rows].copy_(ids_device[: plan.rows], non_blocking=True)
        graph.replay()
        self.replays += 1
        self.passes += 1
        self.replayed_kernels += static.kernels
        eng = self._engine()
        eng.last_h2d_bytes = static.h2d_bytes
        return out[: plan.rows]

    def _record(self, key, plan, ids):
        """Records the pass of `plan` for bucket `key`. Raises `CaptureFailed` if anything goes wrong
        between the first eager run and the end of the capture; by then the capture has been ended and
        what it made has been dropped, so the stream is usable and the pass can run eagerly
        (Kapel: crates/kapel-cuda/src/graph.rs:107-123, crates/kapel-models/src/model.rs:1169-1181)."""
        eng = self._engine()
        from .. import kernels as K

        graph = None
        try:
            static = StaticBatch(key[0], key[1], len(plan.groups), eng.device, eng.chunk, eng.cache.page_size)
            static.fill(plan, ids)
            # Once eagerly on a side stream (kernels set their attributes, the allocator warms up), then the capture.
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                eng.model.forward(static, eng.cache)
            torch.cuda.current_stream().wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            static.memo.clear()
            before = K.launch_count()
            collecting = gc.isenabled()
            gc.disable()                   # nothing may be destroyed while the stream is capturing
            try:
                with torch.cuda.graph(graph, pool=self.pool):
                    if self.fail_next_captures > 0:
                        self.fail_next_captures -= 1
                        raise RuntimeError("injected: the capture was made to fail")
                    out = eng.model.forward(static, eng.cache)
            finally:
                if collecting:
                    gc.enable()
            static.kernels = K.launch_count() - before
        except Exception as e:
            del graph                       # what the capture made so far goes with it
            static = None
            raise CaptureFailed(f"{type(e).__name__}: {e}") from e
        if self.pool is None:
            self.pool = graph.pool()
        self.graphs[key] = (graph, static, out)

    def run(self, plan, ids) -> Optional[torch.Tensor]:
        """Logits [rows, vocab] of a decode-only plan through a recording, or None if no bucket
        takes it or its bucket cannot be recorded (now): the caller then runs the pass eagerly. A
        recording that fails loses only itself; its bucket is tried again `RETRY_AFTER` passes later.
        The result is a view of the recording's output: use it before the next replay."""
        width = max(g.block_table.shape[1] for g in plan.groups) if plan.groups else 1
        key = self.bucket(plan.rows, width)
        self.passes += 1
        if key is None:
            return None
        eng = self._engine()
        if key not in self.graphs:
            failed_at = self.unrecordable.get(key)
            if failed_at is not None and self.passes - failed_at < RETRY_AFTER:
                return None
            try:
                self._record(key, plan, ids)
            except CaptureFailed as e:
                self.unrecordable[key] = self.passes
                self.failed_captures += 1
                self.last_capture_error = str(e)
                return None
            self.unrecordable.pop(key, None)
        graph, static, out = self.graphs[key]
        static.fill(plan, ids)
        graph.replay()
        self.replays += 1
        self.replayed_kernels += static.kernels
        eng.last_h2d_bytes = static.h2d_bytes
        return out[: plan.rows]


class PromptGraphs:
    """Recordings of passes with prompt portions. A pass is a shape: how many tokens each request
    brings behind how many it has, which rows' logits are wanted, how wide the block tables are. The
    portions of a long prompt under a token budget repeat their shapes from request to request (2,048
    tokens behind 0, behind 2,048, ...), and a pass whose shape was seen before is recorded the second
    time and replayed from then on: the same kernels, launched plainly as in an eager pass, without
    the host's share of each launch and with shorter gaps between them (a 2,048-token pass at Gemma 2
    2B sizes: 8.76 to 7.88 ms). Tiles, key slots and every launch's grid are functions of the shape;
    token ids, positions, lines, block tables and the wanted rows are rewritten in the recording's
    input buffer.

    A pass of one request that wants at most one row (a prompt, or a portion of one) is rounded up to
    a round number of rows first, so that prompts of any length share a few dozen shapes: the rows
    added continue the request's positions, carry token 0, write no key or value (their cache line
    is -1, which the append skips) and are wanted by nobody; a row of the request proper never sees
    them (they lie after it), and the pages they would have seen themselves are absent from the block
    table (-1), which every attention kernel skips. Without a recording a pass of a few hundred
    tokens is bound by the host's launches (a 128-token pass at Gemma 2 2B sizes: 3.8 ms)."""

    MIN_ROWS = 65              # fewer rows are a decoding pass's business
    MOST = 32                  # recordings kept; one more shape runs eagerly

    @staticmethod
    def round_rows(rows: int) -> int:
        step = 32 if rows <= 256 else (64 if rows <= 1024 else 128)
        return -(-rows // step) * step

    @staticmethod
    def padded(plan, rows_to: int, page_size: int):
        """`plan` (one entry) with rows added up to `rows_to`, and its block tables as wide as the
        positions of all these rows take."""
        add = rows_to - plan.rows
        more = np.arange(1, add + 1, dtype=np.int32)
        groups = []
        for g in plan.groups:
            width = max(int(g.block_table.shape[1]), -(-(int(plan.row_count[-1]) + add) // page_size))
            table = np.full((g.block_table.shape[0], width), -1, dtype=np.int32)
            table[:, : g.block_table.shape[1]] = g.block_table
            groups.append(dataclasses.replace(g, lines=np.concatenate([g.lines, np.full(add, -1, np.int32)]), block_table=table))
        return dataclasses.replace(
            plan,
            positions=np.concatenate([plan.positions, plan.positions[-1] + more]).astype(np.int32),
            row_entry=np.concatenate([plan.row_entry, np.zeros(add, np.int32)]).astype(np.int32),
            row_count=np.concatenate([plan.row_count, plan.row_count[-1] + more]).astype(np.int32),
            q_len=np.asarray([rows_to], np.int32), groups=groups, taken=[], native=None, added=[])

    def __init__(self, engine, pool_of: Optional[DecodeGraphs] = None):
        self._engine = weakref.ref(engine)
        self._pool_of = pool_of
        self.pool = None
        self.recorded: Dict[tuple, tuple] = {}
        self.seen: Dict[tuple, int] = {}
        self.replays = 0
        self.replayed_kernels = 0
        self.failed_captures = 0
        self.last_capture_error: Optional[str] = None
        self.unrecordable: Dict[tuple, int] = {}
        self.passes = 0
        # Failure injection on the host, for tests: this many of the next recordings raise inside the capture.
        self.fail_next_captures = 0

    @staticmethod
    def shape_of(plan, want_rows, rounded: bool) -> tuple:
        q_len = tuple(int(n) for n in plan.q_len)
        before = tuple(int(plan.row_count[int(s)]) - 1 for s in plan.q_start)
        # which rows are wanted is data (the gather's indices) when a row count was rounded; else part of the shape
        wanted = (len(want_rows),) if rounded else tuple(int(w) for w in want_rows)
        return q_len, before, rounded, wanted, tuple(tuple(g.block_table.shape) for g in plan.groups)

    def run(self, plan, ids, want_rows) -> Optional[torch.Tensor]:
        """Logits of the pass through a recording of its shape, or None: the caller runs it eagerly.
        The result is a view of the recording's output: use it before the next replay."""
        if plan.rows < self.MIN_ROWS:
            return None
        self.passes += 1
        eng = self._engine()
        # (a part that keeps a state of its own a request would take the added rows for tokens: no rounding then)
        rounded = len(plan.entries) == 1 and len(want_rows) <= 1 and not eng.cache.states
        if rounded:
            plan = self.padded(plan, self.round_rows(plan.rows), eng.cache.page_size)
            ids = list(ids) + [0] * (plan.rows - len(ids))
        key = self.shape_of(plan, want_rows, rounded)
        if key not in self.recorded:
            self.seen[key] = self.seen.get(key, 0) + 1
            if self.seen[key] < 2 or len(self.recorded) >= self.MOST:
                if len(self.seen) > 4096:
                    self.seen.clear()
                return None
            failed_at = self.unrecordable.get(key)
            if failed_at is not None and self.passes - failed_at < RETRY_AFTER:
                return None
            try:
                self._record(key, plan, ids, want_rows)
            except CaptureFailed as e:
                self.unrecordable[key] = self.passes
                self.failed_captures += 1
                self.last_capture_error = str(e)
                return None
            self.unrecordable.pop(key, None)
        graph, static, out, kernels = self.recorded[key]
        fresh = StepBatch(plan, ids, want_rows, eng.device, eng.chunk, into=static.dev)
        static.latest = fresh               # its pinned staging buffer lives until the next pass of this shape
        graph.replay()
        self.replays += 1
        self.replayed_kernels += kernels
        eng.last_h2d_bytes = fresh.h2d_bytes
        return out

    def _record(self, key, plan, ids, want_rows) -> None:
        eng = self._engine()
        from .. import kernels as K

        graph = None
        try:
            static = StepBatch(plan, ids, want_rows, eng.device, eng.chunk)
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                eng.model.forward(static, eng.cache)        # once eagerly: attributes set, allocator warm, tiles planned
            torch.cuda.current_stream().wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            pool = self.pool or (self._pool_of.pool if self._pool_of is not None else None)
            before = K.launch_count()
            collecting = gc.isenabled()
            gc.disable()                   # nothing may be destroyed while the stream is capturing
            try:
                with torch.cuda.graph(graph, pool=pool):
                    if self.fail_next_captures > 0:
                        self.fail_next_captures -= 1
                        raise RuntimeError("injected: the capture was made to fail")
                    out = eng.model.forward(static, eng.cache)
            finally:
                if collecting:
                    gc.enable()
            kernels = K.launch_count() - before
        except Exception as e:
            del graph
            raise CaptureFailed(f"{type(e).__name__}: {e}") from e
        if self.pool is None:
            self.pool = pool or graph.pool()
        self.recorded[key] = (graph, static, out, kernels)
