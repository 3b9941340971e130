"""The step function: a batch of (request, its next tokens) in, logits at the wanted places out.

It runs only the tokens it is given, as one batch, from the cache that earlier steps left:
portions of prompts beside single decoded tokens, cut anywhere. Kapel's counterpart is
`Model::run_batch_with` (crates/kapel-models/src/model.rs:986-1033) over `KvCache::begin`
(crates/kapel-models/src/cache.rs:822-842). Lengths move only once the step's kernels are
enqueued; if anything fails before, the pages the plan took go back.
"""
from __future__ import annotations

import itertools
import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Hashable, List, Optional, Sequence, Tuple

import torch

from .. import kernels as K
from ..cache import CacheFull, CacheManager
from ..config import config_from_dir, config_from_json
from ..parts import BuildContext
from ..weights import RandomSource, check_names, open_weights
from .batch import StepBatch
from .model import ModelParts

PAGE_SIZE = 16           # positions a page; Kapel's PAGE (crates/kapel-models/src/cache.rs:49)

_DTYPES = {
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
    "float32": torch.float32, "f32": torch.float32, "fp32": torch.float32,
}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype {name} is not bfloat16 or float32")
        return name
    try:
        return _DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"dtype {name!r} is not one of {sorted(_DTYPES)}") from None


@dataclass
class StepEntry:
    """A request's next tokens and the places among them whose logits are wanted."""

    id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=list)


def require_device() -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError("kapel_b200 runs on a CUDA device (sm_100a); none is available and there is no CPU path")
    K.library()
    return torch.device("cuda", torch.cuda.current_device())


class Engine:
    """A loaded model, its cache and its step function.

    `max_tokens` sizes every group's page pool (ceil(max_tokens / page) pages); `max_sequences`
    the slots. `dtype` "bfloat16" runs the serving kernels, "float32" everything in true 32-bit.
    """

    def __init__(self, config, tensors, dtype="bfloat16", max_tokens: int = 8192, max_sequences: int = 64,
                 device: Optional[torch.device] = None, pages: Optional[int] = None, raw_config: Optional[dict] = None,
                 graphs: bool = True, strict: bool = False):
        self.device = device or require_device()
        self.dtype = parse_dtype(dtype)
        self.config = config
        self.raw_config = raw_config
        self.spec = config.to_spec()
        ctx = BuildContext(dtype=self.dtype, device=self.device, page_size=PAGE_SIZE)
        self.ctx = ctx
        self.model = ModelParts(self.spec, ctx)
        # `tensors` is a mapping from name to tensor: a dict of device tensors, or a source that reads
        # (or makes) a tensor when it is asked for. Names and shapes are checked before anything is
        # read; tensors the model does not name are an error only when `strict`.
        expected = self.model.expected_tensors()
        if hasattr(tensors, "check"):
            self.unexpected_tensors = list(tensors.check(expected, strict))
        else:
            self.unexpected_tensors = check_names(expected, {n: tuple(t.shape) for n, t in tensors.items()},
                                                  "the given tensors", strict)
        self.model.load(tensors)
        ctx.prepared.clear()               # the parts hold what they use
        n_pages = pages if pages is not None else -(-max_tokens // PAGE_SIZE)
        self.cache = CacheManager(
            self.model.cache_needs(), PAGE_SIZE, n_pages, max_sequences,
            allocate=self._allocate, dtype=self.dtype,
        )
        self.chunk = K.attention_chunk()
        self.steps = 0
        self.last_h2d_bytes = 0
        self._request_ids = itertools.count()
        from .graph import DecodeGraphs, PromptGraphs

        self.graphs = DecodeGraphs(self, max_sequences) if (graphs and self.model.graph_safe()) else None
        self.prompt_graphs = PromptGraphs(self, self.graphs) if self.graphs is not None else None

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_dir(cls, folder, dtype="bfloat16", **kw) -> "Engine":
        config, raw = config_from_dir(folder)
        device = kw.pop("device", None) or require_device()
        source = open_weights(folder, device)
        try:
            return cls(config, source, dtype=dtype, device=device, raw_config=raw, **kw)
        finally:
            source.close()

    @classmethod
    def random(cls, config, seed: int = 0, dtype="bfloat16", **kw) -> "Engine":
        """A model of `config` (a typed configuration or config.json's dict) with random weights
        made on the device; for timing, where only the shapes matter."""
        if isinstance(config, dict):
            config = config_from_json(config)
        device = kw.pop("device", None) or require_device()
        return cls(config, RandomSource(config, seed, device=device), dtype=dtype, device=device, raw_config=config.to_json(), **kw)

    def _allocate(self, shape, dtype):
        if isinstance(dtype, str):
            dtype = getattr(torch, dtype)
        return torch.zeros(shape, dtype=dtype, device=self.device)

    # ------------------------------------------------------------------ the step
    @property
    def vocab_size(self) -> int:
        return self.spec.vocab_size

    def _validate(self, entries: Sequence[StepEntry]):
        ids: List[int] = []
        want_rows: List[int] = []
        counts: List[Tuple[Hashable, int]] = []
        vocab = self.spec.vocab_size
        for e in entries:
            n = len(e.tokens)
            if n == 0:
                raise ValueError(f"request {e.id!r} brings no token")
            for t in e.tokens:
                if not 0 <= int(t) < vocab:
                    raise ValueError(f"request {e.id!r}: token {t} is outside the vocabulary (0..{vocab - 1})")
            for w in e.want:
                if not 0 <= int(w) < n:
                    raise ValueError(f"request {e.id!r}: wanted place {w} is outside its {n} tokens")
                want_rows.append(len(ids) + int(w))
            ids.extend(int(t) for t in e.tokens)
            counts.append((e.id, n))
        return ids, want_rows, counts

    def plan(self, entries: Sequence[StepEntry]):
        """Checks the entries, admits new requests into the cache and takes the step's pages."""
        ids, want_rows, counts = self._validate(entries)
        limit = self.spec.max_positions
        added = []
        try:
            for seq_id, n in counts:
                if seq_id not in self.cache:
                    self.cache.add_sequence(seq_id)
                    added.append(seq_id)
                if limit is not None and self.cache.length(seq_id) + n > limit:
                    raise ValueError(
                        f"request {seq_id!r} would reach {self.cache.length(seq_id) + n} positions; the model allows {limit}"
                    )
            plan = self.cache.plan(counts)
        except Exception:
            for seq_id in added:
                self.cache.remove_sequence(seq_id)
            raise
        plan.added = added                 # requests this step brought into the cache: they leave again if it fails
        return plan, ids, want_rows

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Runs one batch; returns float32 logits [number of wanted places, vocab] on the device,
        in the order of the entries and of each entry's `want`.

        The step is enqueued on the current stream and not waited for. The logits of a pass in
        which every request brings one token, or of a pass whose shape was seen before, may be a
        view of a recorded step's output buffer, which the next such pass overwrites: read them (or enqueue what reads them, on the same
        stream) before the next step, or clone them. A caller may enqueue step after step without
        synchronising; the inputs of recorded steps are staged so that this is safe, and the
        host is held back once it is two recorded steps ahead of the device."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        if not entries:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.device)
        plan, ids, want_rows = self.plan(entries)
        try:
            self._clear_fresh_state(plan)
            logits = None
            # A pass of single tokens whose logits are all wanted goes through a recording.
            if self.graphs is not None and plan.rows == len(entries) and len(want_rows) == plan.rows:
                logits = self.graphs.run(plan, ids)
            # A pass with prompt portions whose shape was seen before goes through a recording too.
            if logits is None and self.prompt_graphs is not None and self.graphs is not None:
                logits = self.prompt_graphs.run(plan, ids, want_rows)
            if logits is None:
                batch = StepBatch(plan, ids, want_rows, self.device, self.chunk)
                self.last_h2d_bytes = batch.h2d_bytes
                logits = self.model.forward(batch, self.cache)
        except Exception:
            self.cache.abort(plan)
            for seq_id in getattr(plan, "added", ()):      # a request that came with this step leaves with it
                if seq_id in self.cache:
                    self.cache.remove_sequence(seq_id)
            raise
        self.cache.commit(plan)
        self.steps += 1
        return logits

    # ------------------------------------------------------------------ a pass staged ahead of its tokens
    def prepare_decode(self, seq_ids):
        """Takes the pages and stages the inputs of a pass in which each of `seq_ids` brings one
        token, before the tokens are known (while the pass that chooses them still runs). Returns a
        handle for `step_prepared` / `discard`, or None when such a pass cannot be staged now (no
        recording for its size yet, no pages, a sequence at its limit): then nothing is held."""
        if self.graphs is None or not seq_ids:
            return None
        limit = self.spec.max_positions
        for s in seq_ids:
            if s not in self.cache or (limit is not None and self.cache.length(s) + 1 > limit):
                return None
        try:
            plan = self.cache.plan([(s, 1) for s in seq_ids])
        except CacheFull:
            return None
        if plan.fresh.any():
            self.cache.abort(plan)
            return None
        prepared = self.graphs.prepare(plan)
        if prepared is None:
            self.cache.abort(plan)
        return prepared

    def step_prepared(self, prepared, ids=None, ids_device=None) -> torch.Tensor:
        """Runs a staged pass with its token ids (one a sequence, in the staged order); logits as
        `step` returns them, every row wanted. The ids are a list on the host, or `ids_device`: an
        int32 tensor on the device that a kernel enqueued earlier fills (the tokens the pass before
        chose), so that the pass can be enqueued before the host has seen them."""
        plan = prepared[0]
        vocab = self.spec.vocab_size
        try:
            if ids_device is not None:
                if ids_device.dtype != torch.int32 or ids_device.numel() < plan.rows or ids_device.device != self.device:
                    raise ValueError(f"device ids {tuple(ids_device.shape)} {ids_device.dtype} for a staged pass of {plan.rows}")
            else:
                if len(ids) != plan.rows:
                    raise ValueError(f"{len(ids)} tokens for a staged pass of {plan.rows}")
                for t in ids:
                    if not 0 <= int(t) < vocab:
                        raise ValueError(f"token {t} is outside the vocabulary (0..{vocab - 1})")
            logits = self.graphs.run_prepared(prepared, ids, ids_device)
        except Exception:
            self.cache.abort(plan)
            raise
        self.cache.commit(plan)
        self.steps += 1
        return logits

    def discard(self, prepared) -> None:
        """The staged pass will not run: its pages go back."""
        if prepared is not None and not prepared[0].committed:
            self.cache.abort(prepared[0])

    def _clear_fresh_state(self, plan) -> None:
        if not self.cache.states or not plan.fresh.any():
            return
        host = torch.from_numpy(plan.slots[plan.fresh].astype("int32")).pin_memory()
        slots = host.to(self.device, non_blocking=True)
        for table in self.cache.states.values():
            K.fill_rows(table, slots, 0.0)
        self._fresh_slots_host = host          # pinned memory must outlive its copy

    @property
    def max_positions(self) -> Optional[int]:
        """The most positions a request may reach (config.json's max_position_embeddings), or None."""
        return self.spec.max_positions

    def new_request_ids(self):
        """The counter that every scheduler over this engine draws its request ids from, so that two
        schedulers alive at once never give two requests the same name in the one cache."""
        return self._request_ids

    @property
    def recorded_passes(self) -> int:
        return (self.graphs.replays if self.graphs is not None else 0) + (self.prompt_graphs.replays if self.prompt_graphs is not None else 0)

    def end(self, seq_id) -> None:
        """The request is finished: everything it holds goes back."""
        if seq_id in self.cache:
            self.cache.remove_sequence(seq_id)

    def check(self) -> None:
        """Synchronises and raises if a kernel's bounded wait ever ran out (`kernels.check_async_errors`)."""
        K.check_async_errors()
