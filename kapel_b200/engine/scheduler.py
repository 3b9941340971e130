"""The scheduler above the step function: admit, cut prompts into portions, decode, finish, free.

The policy is Kapel's `Engine` (crates/kapel-infer/src/engine.rs):
  * admission is first come, first served, while the pages that running prompts will still take,
    plus the newcomer's, plus a reserve, fit what is free; alone, a request takes what there is
    (:355-388);
  * a pass holds one token of every decoding request first, then portions of prompts in
    admission order until `max_pass_tokens` is spent (:402-421);
  * a request whose pending tokens all ran in the pass produces a token (:575-580);
  * it ends at an end-of-sequence token (unless `ignore_eos`), at a stop sequence, at
    `max_tokens`, or on an error (:642-660);
  * when pages run out the request admitted last is suspended: its pages go back, it waits at
    the front of the queue, and its prompt and generated tokens are computed again later; a
    request that is alone and still does not fit ends with `CacheFull` (:431-457,392-399);
  * if a pass fails every running request ends (:463-476).
Pages are counted per layer group: a pass fits when every group has the pages it needs.

A model with a limit on positions (`engine.max_positions`, config.json's
max_position_embeddings; Kapel has no such limit) is handled here, not in the step function: a
prompt longer than the limit is refused when it is added, and a request whose next token would
have to be fed beyond the limit ends with "length". The step function's own refusal is thus
never met, and one long request cannot end the others.

The scheduler needs of its engine only `cache` (a CacheManager), `step(entries)`, `end(id)` and
`vocab_size` (and reads `max_positions` and `new_request_ids()` where they exist), so its
decisions are tested on the CPU with a stand-in.
"""
from __future__ import annotations

import itertools
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence

import numpy as np

from ..cache import CacheFull
from ..sampling import Sampler, Sampling, choose_many
from .step import StepEntry


@dataclass
class EngineOptions:
    """Kapel's `EngineOptions` (engine.rs:36-64) without the growing cache and prefix sharing."""

    max_pass_tokens: int = 2048
    max_sequences: int = 256
    reserve: float = 0.0
    # Decoding passes are enqueued one ahead of the host where the tokens can be chosen on the device:
    # the pass after this one is fed the chosen tokens from device memory and starts before the host
    # has read them (this engine's own; Kapel reads every token back before it launches the next pass).
    run_ahead: bool = True


@dataclass
class Request:
    """Kapel's `Request` (crates/kapel-infer/src/generate.rs:72-123), for token ids."""

    prompt: Sequence[int]
    sampling: Sampling = field(default_factory=Sampling)
    max_tokens: int = 256
    eos_ids: Sequence[int] = ()
    ignore_eos: bool = False
    stop: Sequence[Sequence[int]] = ()          # token sequences that end the answer


@dataclass
class Event:
    id: int
    token: Optional[int]
    finish: Optional[str] = None                # "eos", "stop", "length", "error"
    error: Optional[str] = None


@dataclass
class EngineStats:
    """Kapel's `EngineStats` (engine.rs:104-121), pages per layer group."""

    waiting: int = 0
    running: int = 0
    pages: List[int] = field(default_factory=list)
    free_pages: List[int] = field(default_factory=list)
    preemptions: int = 0
    passes: int = 0
    recorded_passes: int = 0
    released_pages: int = 0


class _Entry:
    __slots__ = ("request", "sequence", "prompt_len", "sampler", "running", "generated")

    def __init__(self, request: Request):
        self.request = request
        self.sequence: List[int] = [int(t) for t in request.prompt]
        self.prompt_len = len(self.sequence)
        self.sampler = Sampler(request.sampling)
        self.running = False
        self.generated = 0


class Scheduler:
    def __init__(self, engine, options: Optional[EngineOptions] = None):
        self.engine = engine
        self.cache = engine.cache
        self.options = options or EngineOptions()
        self.entries: Dict[int, _Entry] = {}
        self.waiting: Deque[int] = deque()
        self.running: List[int] = []
        # Request ids name sequences in the engine's one cache, so every scheduler over an engine
        # draws them from the engine's counter: two schedulers alive at once (a stream not yet
        # exhausted beside another call, a user's scheduler beside generate()) never share a name.
        ids = getattr(engine, "new_request_ids", None)
        if ids is not None:
            self._ids = ids()
        else:
            self._ids = getattr(engine, "_request_ids", None) or itertools.count()
            try:
                engine._request_ids = self._ids
            except AttributeError:
                pass
        self.limit = getattr(engine, "max_positions", None)
        self.preemptions = 0
        self.passes = 0
        self.staged = None            # (request ids, engine handle) of a decode pass staged ahead of its tokens
        self.staged_passes = 0        # passes that ran from a staged plan
        self.ahead = None             # (request ids, logits) of a pass already enqueued whose tokens are not chosen yet
        self.ahead_passes = 0         # passes that were enqueued before the host had the tokens they feed
        self._token_host = None       # pinned memory the chosen tokens are copied to, and the event behind the copy
        self._token_event = None

    # ------------------------------------------------------------------ requests
    def add(self, request: Request) -> int:
        if len(request.prompt) == 0:
            raise ValueError("a request needs at least one prompt token")
        vocab = self.engine.vocab_size
        for t in request.prompt:
            if not 0 <= int(t) < vocab:
                raise ValueError(f"prompt token {t} is outside the vocabulary (0..{vocab - 1})")
        if self.limit is not None and len(request.prompt) > self.limit:
            raise ValueError(f"a prompt of {len(request.prompt)} tokens is longer than the {self.limit} positions the model allows")
        rid = next(self._ids)
        self.entries[rid] = _Entry(request)
        self.waiting.append(rid)
        return rid

    def cancel(self, rid: int) -> None:
        """Ends a request wherever it is; its pages go back (engine.rs:308-318)."""
        entry = self.entries.pop(rid, None)
        if entry is None:
            return
        if entry.running:
            self.running.remove(rid)
            self.engine.end(rid)
        else:
            try:
                self.waiting.remove(rid)
            except ValueError:
                pass

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def stats(self) -> EngineStats:
        return EngineStats(
            waiting=len(self.waiting), running=len(self.running), pages=self.cache.total_pages(),
            free_pages=self.cache.free_pages(), preemptions=self.preemptions, passes=self.passes,
            recorded_passes=getattr(self.engine, "recorded_passes", 0), released_pages=self.cache.released_pages,
        )

    # ------------------------------------------------------------------ arithmetic
    def _cached(self, rid: int) -> int:
        return self.cache.length(rid) if rid in self.cache else 0

    def _pending(self, rid: int) -> int:
        return len(self.entries[rid].sequence) - self._cached(rid)

    def _peak_need(self, rid: int, tokens: int) -> List[int]:
        """Pages each group must still give for `tokens` more positions of `rid`. A windowed
        group never holds more than its window plus one pass at a time, whatever the length."""
        need = self.cache.pages_needed(rid, tokens)
        page = self.cache.page_size
        for g, group in enumerate(self.cache.groups):
            if group.window is not None:
                cap = -(-(group.window + self.options.max_pass_tokens) // page) + 1
                need[g] = min(need[g], cap)
        return need

    # ------------------------------------------------------------------ admission
    def _admit(self) -> List[Event]:
        events: List[Event] = []
        if not self.waiting:                                # nobody to admit: nothing to count
            return events
        if len(self.running) >= self.options.max_sequences or self.cache.free_slots() <= 0:
            return events                                   # no slot to admit into either
        n_groups = len(self.cache.groups)
        promised = [0] * n_groups
        for rid in self.running:
            for g, n in enumerate(self._peak_need(rid, self._pending(rid) + 1)):
                promised[g] += n
        total = self.cache.total_pages()
        margin = [int(np.ceil(self.options.reserve * t)) for t in total]
        while self.waiting and len(self.running) < self.options.max_sequences and self.cache.free_slots() > 0:
            rid = self.waiting[0]
            entry = self.entries[rid]
            needed = self._peak_need(rid, len(entry.sequence) + 1)
            free = self.cache.free_pages()
            fits = all(promised[g] + needed[g] + margin[g] <= free[g] for g in range(n_groups))
            alone = not self.running and all(needed[g] <= free[g] for g in range(n_groups))
            if not (fits or alone):
                if not self.running and any(needed[g] > total[g] for g in range(n_groups)):
                    # It could never run, even alone in an empty cache: end it instead of waiting forever.
                    self.waiting.popleft()
                    del self.entries[rid]
                    g = next(g for g in range(n_groups) if needed[g] > total[g])
                    events.append(Event(rid, None, "error", str(CacheFull(needed[g], total[g], self.cache.groups[g].name))))
                    continue
                break
            for g in range(n_groups):
                promised[g] += needed[g]
            self.waiting.popleft()
            self.cache.add_sequence(rid)
            entry.running = True
            self.running.append(rid)
        return events

    def _suspend_last(self) -> None:
        rid = self.running.pop()
        self.entries[rid].running = False
        self.engine.end(rid)
        self.waiting.appendleft(rid)
        self.preemptions += 1

    def _plan(self) -> List[tuple]:
        budget = max(1, self.options.max_pass_tokens)
        out = []
        for rid in self.running:
            if self._pending(rid) == 1:
                out.append((rid, 1))
                budget = max(0, budget - 1)
        for rid in self.running:
            pending = self._pending(rid)
            if pending > 1 and budget > 0:
                count = min(pending, budget)
                out.append((rid, count))
                budget -= count
        return out

    # ------------------------------------------------------------------ one pass
    def step(self) -> List[Event]:
        """One pass of the model: a token of every decoding request and portions of prompts.
        Returns the tokens it gave and the requests that ended; nothing when there is no work."""
        events = self._admit()
        ahead, self.ahead = self.ahead, None
        if ahead is not None:
            # This pass is already on its way (enqueued while the host still read the tokens before).
            return self._after_launch(events, *ahead)
        staged, self.staged = self.staged, None
        if staged is not None:
            # The pass staged while the last one ran is this pass if nothing changed since: the same
            # requests run, each with exactly its new token to feed.
            rids, handle = staged
            if rids == self.running and all(self._pending(r) == 1 for r in rids):
                return self._finish_staged(events, rids, handle)
            self._discard(handle)
        while True:
            pass_ = self._plan()
            need = [0] * len(self.cache.groups)
            for rid, count in pass_:
                for g, n in enumerate(self.cache.pages_needed(rid, count)):
                    need[g] += n
            free = self.cache.free_pages()
            short = [g for g in range(len(need)) if need[g] > free[g]]
            if not short:
                break
            if len(self.running) == 1:
                rid = self.running[0]
                g = short[0]
                error = CacheFull(need[g], free[g], self.cache.groups[g].name)
                self.cancel(rid)
                events.append(Event(rid, None, "error", str(error)))
                return events
            self._suspend_last()
        if not pass_:
            return events
        return self._finish_pass(events, pass_)

    def settle(self) -> List[Event]:
        """Ends what runs ahead of the host: reads the pass that is already on its way (and gives its
        tokens, as `step` would have), and gives back the pages of a pass that was staged. After it
        the engine's cache holds every running request's tokens but the last, which is the one to
        feed next; somebody who then steps the engine directly sees a consistent state."""
        events: List[Event] = []
        ahead, self.ahead = self.ahead, None
        if ahead is not None:
            rids, logits = ahead
            try:
                rows = [i for i, r in enumerate(rids) if r in self.entries and self.entries[r].running]
                producing = [rids[i] for i in rows]
                tokens = self._choose(logits, producing, rows)
            except Exception as e:
                return self._fail_pass(events, e)
            events = self._give(events, producing, tokens)
        staged, self.staged = self.staged, None
        if staged is not None:
            self._discard(staged[1])
        return events

    def _discard(self, handle) -> None:
        discard = getattr(self.engine, "discard", None)
        if discard is not None:
            discard(handle)

    def _stage_next(self, pass_, producing) -> None:
        """While the pass just launched runs: if it was decoding only and every request is sure to
        go on unless it meets an end-of-sequence or stop token, take the next pass's pages and
        write its inputs now, so that only the token ids remain to be filled in."""
        prepare = getattr(self.engine, "prepare_decode", None)
        if prepare is None or len(producing) != len(pass_) or [r for r, _ in pass_] != self.running:
            return
        # A waiting request joins the next pass only if it can be admitted: with every slot taken it
        # cannot be until a request ends, and a pass staged for a request that then ends is handled.
        if self.waiting and len(self.running) < self.options.max_sequences and self.cache.free_slots() > 0:
            return
        for rid in producing:
            entry = self.entries[rid]
            if entry.generated + 1 >= entry.request.max_tokens:
                return
            if self.limit is not None and len(entry.sequence) + 1 > self.limit:
                return
        handle = prepare(list(self.running))
        if handle is not None:
            self.staged = (list(self.running), handle)

    def _finish_staged(self, events, rids, handle) -> List[Event]:
        """The staged pass: each request feeds its newest token and gets the next."""
        try:
            logits = self.engine.step_prepared(handle, [self.entries[r].sequence[-1] for r in rids])
            self.staged_passes += 1
            self.passes += 1
        except Exception as e:                      # the pass failed: every running request ends
            return self._fail_pass(events, e)
        return self._after_launch(events, rids, logits)

    def _after_launch(self, events, rids, logits) -> List[Event]:
        """A pass of one token for each of `rids` has been enqueued and `logits` (a row a request, in
        that order) will hold its result. Stages the pass after it; chooses the tokens; and, where
        they can be chosen on the device, enqueues the staged pass with the tokens fed from device
        memory before the host waits for them. A request that ended or was cancelled since the pass
        was enqueued has a row nobody reads."""
        try:
            rows = [i for i, r in enumerate(rids) if r in self.entries and self.entries[r].running]
            producing = [rids[i] for i in rows]
            whole = len(producing) == len(rids)
            if whole:
                self._stage_next([(r, 1) for r in rids], producing)
            tokens = None
            if whole and self.staged is not None and self.options.run_ahead and hasattr(self.engine, "step_prepared"):
                chosen = self._choose_on_device(logits, producing, rows)
                if chosen is not None:
                    import torch

                    if self._token_host is None or self._token_host.numel() < chosen.numel():
                        self._token_host = torch.empty((max(256, chosen.numel()),), dtype=torch.int32).pin_memory()
                        self._token_event = torch.cuda.Event()
                    self._token_host[: chosen.numel()].copy_(chosen, non_blocking=True)
                    self._token_event.record()
                    next_rids, handle = self.staged
                    self.staged = None
                    ahead_logits = self.engine.step_prepared(handle, ids_device=chosen)     # enqueued behind the copy
                    self.staged_passes += 1
                    self.ahead_passes += 1
                    self.passes += 1
                    self.ahead = (next_rids, ahead_logits)
                    self._token_event.synchronize()                                         # the pass just enqueued runs meanwhile
                    host = self._token_host[: chosen.numel()].tolist()
                    tokens = [host[i] for i in rows]
            if tokens is None:
                tokens = self._choose(logits, producing, rows)
        except Exception as e:                      # the pass failed: every running request ends
            return self._fail_pass(events, e)
        return self._give(events, producing, tokens)

    def _fail_pass(self, events, e) -> List[Event]:
        self.ahead = None                           # a pass on its way is left to finish; nobody reads its rows
        staged, self.staged = self.staged, None
        if staged is not None:
            self._discard(staged[1])
        for rid in list(self.running):
            self.cancel(rid)
            events.append(Event(rid, None, "error", f"{type(e).__name__}: {e}"))
        return events

    def _give(self, events, producing, tokens) -> List[Event]:
        for rid, token in zip(producing, tokens):
            entry = self.entries[rid]
            entry.sequence.append(int(token))
            entry.generated += 1
            finish = self._finish_reason(entry, int(token))
            events.append(Event(rid, int(token), finish))
            if finish is not None:
                self.cancel(rid)
        return events

    def _finish_pass(self, events, pass_) -> List[Event]:
        producing = [rid for rid, count in pass_ if count == self._pending(rid)]
        entries = []
        for rid, count in pass_:
            entry = self.entries[rid]
            at = self._cached(rid)
            tokens = entry.sequence[at : at + count]
            entries.append(StepEntry(rid, tokens, [count - 1] if count == self._pending(rid) else []))
        try:
            logits = self.engine.step(entries)
            self.passes += 1
        except Exception as e:                      # the pass failed: every running request ends
            return self._fail_pass(events, e)
        if len(producing) == len(pass_):
            return self._after_launch(events, producing, logits)        # every request of the pass gets a token: a row each, in order
        try:
            tokens = self._choose(logits, producing)
        except Exception as e:
            return self._fail_pass(events, e)
        return self._give(events, producing, tokens)

    def _finish_reason(self, entry: _Entry, token: int) -> Optional[str]:
        req = entry.request
        if not req.ignore_eos and token in req.eos_ids:
            return "eos"
        generated = entry.sequence[entry.prompt_len:]
        for stop in req.stop:
            n = len(stop)
            if n and len(generated) >= n and list(generated[-n:]) == [int(t) for t in stop]:
                return "stop"
        if entry.generated >= req.max_tokens:
            return "length"
        if self.limit is not None and len(entry.sequence) > self.limit:
            return "length"                 # the token just given would have to be fed at a position beyond the limit
        return None

    # ------------------------------------------------------------------ choosing tokens
    def _choose_on_device(self, logits, producing: List[int], rows: List[int]):
        """The chosen tokens as an int32 device tensor, a token a row of `logits` (rows outside `rows`
        belong to nobody and get the largest logit), enqueued and not waited for; None where the
        choice needs the host (filters, penalties) or the logits are not on a device."""
        if not producing or not getattr(logits, "is_cuda", False):
            return None
        entries = [self.entries[rid] for rid in producing]
        if not all(e.request.sampling.on_device() for e in entries):
            return None
        import torch

        from .. import kernels as K

        if all(e.request.sampling.is_greedy() for e in entries):
            return K.sample(logits)
        n = int(logits.shape[0])
        temps, us = [0.0] * n, [0.0] * n
        for i, e in zip(rows, entries):
            temps[i] = max(0.0, e.request.sampling.temperature)
            us[i] = e.sampler.uniform() if temps[i] > 0 else 0.0
        host = torch.tensor([temps, us], dtype=torch.float32).pin_memory()
        dev = host.to(logits.device, non_blocking=True)
        self._sample_inputs = host                  # pinned memory must outlive its copy
        return K.sample(logits, dev[0], dev[1])

    def _choose(self, logits, producing: List[int], rows: Optional[List[int]] = None) -> List[int]:
        """One token per producing request: on the device when only the logits decide (greedy
        without penalties, or a plain temperature; engine.rs:584-597), else on the host in
        64-bit with the request's own sampler (engine.rs:599-616). `rows` names each request's
        row of `logits` (by default row i is request i's)."""
        if not producing:
            return []
        rows = list(range(len(producing))) if rows is None else rows
        chosen = self._choose_on_device(logits, producing, rows)
        if chosen is not None:
            host = chosen.cpu().tolist()
            return [host[i] for i in rows]
        entries = [self.entries[rid] for rid in producing]
        table = logits.detach().cpu().numpy() if hasattr(logits, "detach") else np.asarray(logits)
        if len(rows) != table.shape[0] or rows != list(range(table.shape[0])):
            table = table[rows]
        return choose_many([e.sampler for e in entries], table, [e.sequence for e in entries], [e.prompt_len for e in entries])
