"""Choosing the next token: Kapel's options, order and generator.

Order (crates/kapel-infer/src/sampling.rs:5-8,157-238): frequency and presence penalties, the
repetition penalty, then greedy if the temperature is 0, else temperature, top_k, top_p, min_p,
then a draw from what is left. The generator is xoshiro256** seeded by four SplitMix64 outputs
(sampling.rs:91-121); a draw is the first index whose running total of probabilities exceeds a
uniform number in [0, 1) (sampling.rs:241-260). Arithmetic on the host is 64-bit, as there.

A request whose choice needs only the logits (greedy without penalties, or a plain
temperature) can be served where the logits are, by `kernels.sample`; the uniform number still
comes from this generator, so the same seed gives the same tokens.

The arithmetic runs in the host library (`csrc/host/sampler_core.cpp`): a choice over 256,000
logits with top_k takes about a millisecond there, where sorting them with numpy took ten to
forty, and `choose_many` serves the requests of a step on several threads.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np

from ..hostlib import host_library

_M = (1 << 64) - 1
_CPUS = os.cpu_count() or 1


@dataclass
class Sampling:
    """Kapel's `Sampling` (crates/kapel-infer/src/sampling.rs:10-50), same names and defaults."""

    temperature: float = 0.0
    top_k: Optional[int] = None
    top_p: float = 1.0
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    seed: int = 0

    @classmethod
    def greedy(cls) -> "Sampling":
        return cls()

    @classmethod
    def from_generation_config(cls, config: dict) -> "Sampling":
        """generation_config.json with the defaults Kapel takes for what it leaves out: greedy
        unless do_sample; then temperature 1 and top_k 50 (sampling.rs:61-78)."""
        s = cls(repetition_penalty=float(config.get("repetition_penalty") or 1.0))
        if config.get("do_sample") is True:
            s.temperature = float(config["temperature"]) if config.get("temperature") is not None else 1.0
            k = config.get("top_k")
            s.top_k = None if k == 0 else (int(k) if k is not None else 50)
            s.top_p = float(config["top_p"]) if config.get("top_p") is not None else 1.0
            s.min_p = float(config["min_p"]) if config.get("min_p") is not None else 0.0
        return s

    def is_greedy(self) -> bool:
        return self.temperature <= 0.0

    def has_penalties(self) -> bool:
        return self.repetition_penalty != 1.0 or self.frequency_penalty != 0.0 or self.presence_penalty != 0.0

    def has_filters(self) -> bool:
        return (self.top_k is not None and self.top_k > 0) or self.top_p < 1.0 or self.min_p > 0.0

    def is_argmax(self) -> bool:
        """The choice is the most likely token whatever the sequence (sampling.rs:139-145)."""
        return self.is_greedy() and not self.has_penalties()

    def on_device(self) -> bool:
        """Only the logits, a temperature and a uniform number decide."""
        return not self.has_penalties() and (self.is_greedy() or not self.has_filters())


class Rng:
    """xoshiro256**, seeded through SplitMix64: the same numbers on every machine. The four words
    of state live where the host library can advance them too."""

    def __init__(self, seed: int):
        self._lib = host_library()
        self.state = np.zeros(4, np.uint64)
        self._ptr = self.state.ctypes.data                  # the array is never replaced, only written
        self._lib.ks_seed(seed & _M, self._ptr)

    @property
    def s(self) -> List[int]:
        return self.state.tolist()

    @staticmethod
    def _rotl(x: int, k: int) -> int:
        return ((x << k) | (x >> (64 - k))) & _M

    def next_u64(self) -> int:
        s = self.s
        result = (self._rotl((s[1] * 5) & _M, 7) * 9) & _M
        t = (s[1] << 17) & _M
        s[2] ^= s[0]
        s[3] ^= s[1]
        s[1] ^= s[2]
        s[0] ^= s[3]
        s[2] ^= t
        s[3] = self._rotl(s[3], 45)
        self.state[:] = np.asarray(s, np.uint64)
        return result

    def uniform(self) -> float:
        return self._lib.ks_uniform(self._ptr)


def _row(logits):
    """`logits` as a contiguous float32 or float64 array and the host library's code for its type."""
    a = logits if isinstance(logits, np.ndarray) else np.asarray(logits, dtype=np.float64)
    if a.dtype != np.float32 and a.dtype != np.float64:
        a = a.astype(np.float64)
    a = np.ascontiguousarray(a)
    return a, (0 if a.dtype == np.float32 else 1)


class Sampler:
    """One request's chooser: its settings and its own generator."""

    def __init__(self, settings: Sampling):
        self.settings = settings
        self.rng = Rng(settings.seed)
        s = settings
        self._floats = np.asarray([s.temperature, s.top_p, s.min_p, s.repetition_penalty, s.frequency_penalty, s.presence_penalty], np.float64)
        self._top_k = int(s.top_k) if s.top_k is not None and s.top_k > 0 else 0

    def uniform(self) -> float:
        return self.rng.uniform()

    def _sequence(self, sequence: Sequence[int]) -> np.ndarray:
        """The tokens the penalties look at; none when there are no penalties."""
        if not self.settings.has_penalties() or len(sequence) == 0:
            return np.zeros(0, np.int32)
        return np.asarray(sequence, dtype=np.int64).clip(-1, 2 ** 31 - 1).astype(np.int32)

    def _run(self, logits, sequence, generated_from, probs, want_draw) -> int:
        row, code = _row(logits)
        seq = self._sequence(sequence)
        return self.rng._lib.ks_choose(
            row.ctypes.data, code, row.shape[0], self._floats.ctypes.data, self._top_k, seq.ctypes.data, seq.shape[0],
            int(generated_from), self.rng._ptr, None if probs is None else probs.ctypes.data, want_draw)

    def distribution(self, logits, sequence: Sequence[int], generated_from: int):
        """(token, None) when the choice is certain, else (None, probabilities in 64-bit).
        `sequence` is prompt and generated tokens, the generated ones from index `generated_from`
        on. Nothing is drawn."""
        probs = np.empty(len(logits), np.float64)
        token = self._run(logits, sequence, generated_from, probs, 0)
        return (token, None) if token >= 0 else (None, probs)

    def choose(self, logits, sequence: Sequence[int] = (), generated_from: int = 0) -> int:
        return self._run(logits, sequence, generated_from, None, 1)


def choose_many(samplers: Sequence[Sampler], rows: np.ndarray, sequences: Sequence[Sequence[int]],
                generated_from: Sequence[int], threads: Optional[int] = None) -> List[int]:
    """One token for each sampler from its row of `rows` ([requests, vocabulary], float32 or
    float64), on up to `threads` threads of the host library (default: the requests, at most eight
    and at most the processors). Each request uses only its own generator, so the tokens do not
    depend on the threads."""
    count = len(samplers)
    if count == 0:
        return []
    rows, code = _row(rows)
    if rows.ndim != 2 or rows.shape[0] != count:
        raise ValueError(f"{count} samplers for logits of shape {rows.shape}")
    lib = samplers[0].rng._lib
    floats = np.concatenate([s._floats for s in samplers])
    top_k = np.asarray([s._top_k for s in samplers], np.int32)
    seqs = [s._sequence(q) for s, q in zip(samplers, sequences)]
    seq_ptrs = (ctypes.c_void_p * count)(*[q.ctypes.data for q in seqs])
    seq_lens = np.asarray([q.shape[0] for q in seqs], np.int32)
    gen_from = np.asarray([int(g) for g in generated_from], np.int32)
    states = np.stack([s.rng.state for s in samplers])
    tokens = np.empty(count, np.int32)
    if threads is None:                                     # threads pay from a few hundred thousand logits on
        threads = min(count, 8, _CPUS) if rows.size >= 200_000 else 1
    lib.ks_choose_many(count, rows.ctypes.data, rows.shape[1], code, rows.shape[1], floats.ctypes.data, top_k.ctypes.data,
                       ctypes.addressof(seq_ptrs), seq_lens.ctypes.data, gen_from.ctypes.data, states.ctypes.data,
                       tokens.ctypes.data, int(threads))
    for i, s in enumerate(samplers):
        s.rng.state[:] = states[i]
    return tokens.tolist()
