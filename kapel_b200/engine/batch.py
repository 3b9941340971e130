"""One step's rows on the device: what the cache manager planned, copied over in one piece.

Kapel uploads `ids, positions, lines, pages, rows, slots` as separate small tensors
(crates/kapel-models/src/cache.rs:822-842). Here they are slices of one int32 buffer that
crosses from pinned host memory in a single copy.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache import Plan


class GroupBatch:
    __slots__ = ("lines", "block_table")

    def __init__(self, lines, block_table):
        self.lines = lines                # [rows] int32 on the device
        self.block_table = block_table    # [entries, width] int32 on the device


def _chunks_touched(row_count: np.ndarray, window: Optional[int], chunk: int) -> int:
    """The most key chunks (cut at absolute multiples of `chunk`) any row of the step reads."""
    c = row_count[row_count > 0].astype(np.int64)
    if c.size == 0:
        return 1
    first = np.maximum(0, c - window) if window else np.zeros_like(c)
    return int(((c - 1) // chunk - first // chunk + 1).max())


SPLIT_STEP = 64          # splits are multiples of the kernels' key tile


def decode_split(pairs: int, longest: int, sms: int, window: Optional[int] = None, relative: bool = False):
    """(split, slots) of the decode attention kernel, which runs one block a multiprocessor.
    Keys are cut at multiples of `split`, counted from key 0 (`slots` then covers the longest
    request, `longest` positions) or, with `relative`, from each row's first visible key (`slots`
    covers what a row can see). A row reads at most `window` keys, so only about window / split of the
    slots do work. The split is chosen so that the working blocks (`pairs` (tile, kv head)
    pairs times working slots) take as little time as possible: waves of blocks times the keys a
    block walks plus what a block costs to start and to merge (about 192 keys' worth)."""
    pairs = max(1, pairs)
    span = min(longest, window) if window else longest
    best = None
    most = max(1, -(-span // SPLIT_STEP))
    for want in range(1, min(most, 4 * sms) + 1):
        split = max(SPLIT_STEP, -(-(-(-span // want)) // SPLIT_STEP) * SPLIT_STEP)
        working = -(-span // split) + (1 if (window and longest > window and not relative) else 0)
        cost = -(-(pairs * working) // sms) * (split + 192)
        if best is None or cost < best[0]:
            best = (cost, split)
    split = best[1]
    return split, max(1, -(-(span if relative else longest) // split))


# What a block costs beyond its 64-key steps, what the merge of partial sums costs beyond its traffic
# (both in steps), microseconds a step, and how many multiprocessors a block takes, by prompt kernel;
# from sweeps of the split at Gemma 2 2B head sizes with 2,048 tokens behind 4,096 to 129,024 (a block
# that starts among running ones costs 20 to 27 us before its first and after its last step, twice
# what it costs in a launch of its own). The tcgen05 kernels' steps are short, so their fixed costs
# weigh more and they are cut into slots only when a few tiles face a long history; "tcgen05_pair" is
# the kernel on pairs of blocks (a tile of 256 rows on two multiprocessors, half the time a step).
PROMPT_KERNEL_COSTS = {"mma": (0.5, 1.0, 4.5, 1), "tcgen05": (18.0, 15.0, 1.2, 1), "tcgen05_pair": (32.0, 18.0, 0.85, 2)}


def prompt_costs_of(prompt_kernel: str, head_dim: int, pairs: Optional[int] = None) -> str:
    """The entry of PROMPT_KERNEL_COSTS for the kernel that will run prompt portions of this head size."""
    from .. import kernels as K

    if prompt_kernel == "tcgen05" and K.attention_tile_rows(False, prompt_kernel, head_dim, pairs) > 128:
        return "tcgen05_pair"
    return prompt_kernel


def prompt_split(first_counts, last_counts, pairs_per_tile: int, sms: int, window: Optional[int], rows: int, hq: int, d: int,
                 kernel: str = "mma"):
    """(split, slots) of the prompt attention kernel. A tile of a long prompt walks all the keys
    before it, so late tiles work many times longer than early ones; cutting the keys into slots
    of `split` positions evens the blocks out at the price of partial sums that a second kernel
    merges. The choice minimises an estimate of the time: the longest block or the mean load of a
    multiprocessor, whichever is larger, plus the merge, all counted in 64-key steps."""
    block_cost, merge_cost, step_us, sms_a_block = PROMPT_KERNEL_COSTS[kernel]
    sms = max(1, sms // sms_a_block)                     # blocks (or pairs of blocks) that run at once
    first = np.asarray(first_counts, np.int64)
    last = np.asarray(last_counts, np.int64)
    lo = np.maximum(0, first - window) if window else np.zeros_like(first)
    longest = int(last.max()) if last.size else 0
    best = None
    for split in (0, 4096, 2048, 1024, 512, 256, 128):
        if split == 0:
            steps = -(-(last - lo // 64 * 64) // 64)
            work = steps.astype(np.float64)
            slots = 1
            merge = 0.0
        else:
            if split >= longest:
                continue
            slots = -(-longest // split)
            z = np.arange(slots)[None, :]
            a = np.maximum(lo[:, None], z * split)
            b = np.minimum(last[:, None], (z + 1) * split)
            steps = np.where(b > a, -(-(b - a // 64 * 64) // 64), 0)
            work = steps.astype(np.float64).reshape(-1)
            # what the partial sums cost to write and read back (at ~5 TB/s), in steps, plus a launch
            merge = merge_cost + slots * rows * hq * (d + 2) * 8 / 5e12 / (step_us * 1e-6)
        work = work[work > 0] + block_cost               # what it costs to start and finish a block
        if work.size == 0:
            continue
        cost = max(float(work.max()), float(work.sum()) * pairs_per_tile / sms * 1.1) + merge
        if best is None or cost < best[0]:
            best = (cost, split, slots)
    return (best[1], best[2]) if best else (0, 1)


_SMS = {}


def sm_count(device) -> int:
    key = str(device)
    if key not in _SMS:
        _SMS[key] = torch.cuda.get_device_properties(device).multi_processor_count if torch.device(device).type == "cuda" else 148
    return _SMS[key]


def cut_tiles(q_start, q_len, tokens_per_tile: int):
    """(tile_entry, tile_row0, tile_nq): each request's rows in runs of at most `tokens_per_tile`."""
    entry, row0, nq = [], [], []
    for e, (start, n) in enumerate(zip(q_start.tolist(), q_len.tolist())):
        for at in range(0, n, tokens_per_tile):
            entry.append(e)
            row0.append(start + at)
            nq.append(min(tokens_per_tile, n - at))
    return np.asarray(entry, np.int32), np.asarray(row0, np.int32), np.asarray(nq, np.int32)


class StepBatch:
    """Device views of a step. `memo` holds what parts share within the step (rotary tables)."""

    def __init__(self, plan: Plan, ids: Sequence[int], want_rows: Sequence[int], device, chunk: int,
                 fixed_slots: Optional[int] = None, into: Optional[torch.Tensor] = None):
        """`into`: a device buffer of a recorded pass of the same shape (the same number of values), to
        be rewritten in place instead of a new one."""
        self.plan = plan
        self.rows = plan.rows
        self.entries = len(plan.entries)
        self.chunk = chunk
        self.fixed_slots = fixed_slots
        self.memo: Dict[object, object] = {}
        self._slots_memo: Dict[Optional[int], int] = {}
        parts: List[np.ndarray] = [
            np.asarray(ids, np.int32), plan.positions, plan.row_entry, plan.row_count,
            np.asarray(want_rows, np.int32), plan.slots,
        ]
        for g in plan.groups:
            parts.append(g.lines)
            parts.append(g.block_table.reshape(-1))
        sizes = [p.size for p in parts]
        total = sum(sizes)
        host = torch.empty((max(total, 1),), dtype=torch.int32, pin_memory=(device.type == "cuda"))
        flat = host.numpy()
        at = 0
        for p in parts:
            flat[at : at + p.size] = p
            at += p.size
        self.h2d_bytes = total * 4
        if into is not None:
            if into.numel() != host.numel():
                raise ValueError(f"a recorded pass of {into.numel()} input values was offered a pass of {host.numel()}")
            into.copy_(host, non_blocking=True)
            dev = into
        else:
            dev = host.to(device, non_blocking=True)
        self.dev = dev
        self.sizes = sizes
        self._host = host                 # keeps the pinned buffer alive until the copy is done
        self._assign(dev, sizes, [g.block_table.shape for g in plan.groups])

    def _assign(self, dev, sizes, table_shapes):
        views, at = [], 0
        for n in sizes:
            views.append(dev[at : at + n])
            at += n
        self.ids, self.positions, self.row_entry, self.row_count, self.want_rows, self.slots = views[:6]
        self.groups = []
        for i, shape in enumerate(table_shapes):
            self.groups.append(GroupBatch(views[6 + 2 * i], views[7 + 2 * i].view(shape)))

    def attention_tiles(self, heads_per_kv: int, kv_heads: int, window: Optional[int] = None, head_dim: int = 256,
                        prompt_kernel: str = "mma"):
        """How the tensor-core attention kernel cuts this step: (decode, (tile_entry, tile_row0,
        tile_nq) on the device, split, slots). `decode` is the most rows (tokens x query heads of a
        kv head) of any request when that is at most 16, which selects the decode kernel, else 0.
        The keys are split across blocks when the tiles alone are too few to fill the GPU;
        `prompt_kernel` names the kernel whose costs decide that for prompt portions. A fifth
        value says whether the slots are counted from each row's first visible key (every
        request brings one token) or from key 0."""
        key = ("tiles", heads_per_kv, kv_heads, window, head_dim, prompt_kernel)
        if key not in self.memo:
            from .. import kernels as K

            plan = self.plan
            pairs = K.prompt_pairs(plan.rows, int(plan.row_count.max()))
            self.pairs = pairs                              # the attention part hands it to the kernel
            costs_of = prompt_costs_of(prompt_kernel, head_dim, pairs)
            most = int(plan.q_len.max()) * heads_per_kv
            decode = most if most <= K.attention_mma_rows(True) else 0      # rows a tile in decode mode, else 0
            per_tile = max(1, K.attention_tile_rows(bool(decode), prompt_kernel, head_dim, pairs) // heads_per_kv)
            arrays = cut_tiles(plan.q_start, plan.q_len, per_tile)
            n = arrays[0].size
            host = torch.from_numpy(np.concatenate(arrays)).pin_memory() if self.ids.is_cuda else torch.from_numpy(np.concatenate(arrays))
            dev = host.to(self.ids.device, non_blocking=True)
            tiles = (dev[:n], dev[n : 2 * n], dev[2 * n :])
            longest = int(plan.row_count.max())
            relative = bool(decode) and int(plan.q_len.max()) == 1
            if decode:
                split, slots = decode_split(n * kv_heads, longest, sm_count(self.ids.device), window, relative)
            else:
                firsts = plan.row_count[arrays[1]]
                split, slots = prompt_split(firsts, firsts + arrays[2] - 1, kv_heads, sm_count(self.ids.device), window,
                                            plan.rows, heads_per_kv * kv_heads, head_dim, costs_of)
            self.memo[key] = (decode, tiles, split, slots, relative, host)
        return self.memo[key][:5]

    def attention_slots(self, window: Optional[int]) -> int:
        """Chunk slots the row-wise attention kernel needs for a layer with this window."""
        if window not in self._slots_memo:
            if self.fixed_slots is not None:
                n = self.fixed_slots
                if window:
                    n = min(n, (window - 1) // self.chunk + 2)
            else:
                n = _chunks_touched(self.plan.row_count, window, self.chunk)
            self._slots_memo[window] = max(1, n)
        return self._slots_memo[window]
