"""Choosing the next token: Kapel's options, order and generator.

Order (crates/kapel-infer/src/sampling.rs:5-8,157-238): frequency and presence penalties, the
repetition penalty, then greedy if the temperature is 0, else temperature, top_k, top_p, min_p,
then a draw from what is left. The generator is xoshiro256** seeded by four SplitMix64 outputs
(sampling.rs:91-121); a draw is the first index whose running total of probabilities exceeds a
uniform number in [0, 1) (sampling.rs:241-260). Arithmetic on the host is 64-bit, as there.

A request whose choice needs only the logits (greedy without penalties, or a plain
temperature) can be served where the logits are, by `kernels.sample`; the uniform number still
comes from this generator, so the same seed gives the same tokens.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np

_M = (1 << 64) - 1


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
    """xoshiro256**, seeded through SplitMix64: the same numbers on every machine."""

    def __init__(self, seed: int):
        z = seed & _M
        s = []
        for _ in range(4):
            z = (z + 0x9E3779B97F4A7C15) & _M
            x = z
            x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _M
            x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _M
            s.append(x ^ (x >> 31))
        self.s = s

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
        return result

    def uniform(self) -> float:
        return (self.next_u64() >> 11) / float(1 << 53)


def argmax(values: np.ndarray) -> int:
    """The first largest; a NaN never, unless all are (sampling.rs:291-299)."""
    ok = ~np.isnan(values)
    if not ok.any():
        return 0
    return int(np.argmax(np.where(ok, values, -np.inf)))


def softmax(logits: np.ndarray) -> np.ndarray:
    m = np.max(logits)
    if m == -np.inf or np.isnan(m):
        return np.zeros_like(logits)
    e = np.exp(logits - m)
    return e / e.sum()


class Sampler:
    """One request's chooser: its settings and its own generator."""

    def __init__(self, settings: Sampling):
        self.settings = settings
        self.rng = Rng(settings.seed)

    def uniform(self) -> float:
        return self.rng.uniform()

    def distribution(self, logits: np.ndarray, sequence: Sequence[int], generated_from: int):
        """(token, None) when the choice is certain, else (None, probabilities). `logits` is a
        float64 array that this call changes; `sequence` is prompt and generated tokens, the
        generated ones from index `generated_from` on."""
        s = self.settings
        n = logits.shape[0]
        if s.frequency_penalty != 0.0 or s.presence_penalty != 0.0:
            counts = {}
            for t in sequence[min(generated_from, len(sequence)):]:
                counts[t] = counts.get(t, 0) + 1
            for t, c in counts.items():
                if 0 <= t < n:
                    logits[t] -= c * s.frequency_penalty + s.presence_penalty
        if s.repetition_penalty != 1.0:
            for t in set(sequence):
                if 0 <= t < n:
                    logits[t] = logits[t] * s.repetition_penalty if logits[t] < 0 else logits[t] / s.repetition_penalty
        if s.is_greedy():
            return argmax(logits), None
        logits /= s.temperature
        if s.top_k is not None and 0 < s.top_k < n:
            kth = np.sort(logits)[::-1][s.top_k - 1]
            logits[logits < kth] = -np.inf
        if s.top_p < 1.0:
            probs = softmax(logits)
            order = np.lexsort((np.arange(n), -probs))        # by probability, then by index
            before = np.concatenate(([0.0], np.cumsum(probs[order])[:-1]))
            logits[order[before >= s.top_p]] = -np.inf
        if s.min_p > 0.0:
            probs = softmax(logits)
            logits[probs < s.min_p * probs.max()] = -np.inf
        probs = softmax(logits)
        if not (probs > 0).any():
            return argmax(logits), None
        return None, probs

    def choose(self, logits, sequence: Sequence[int] = (), generated_from: int = 0) -> int:
        token, probs = self.distribution(np.array(logits, dtype=np.float64), sequence, generated_from)
        if token is not None:
            return token
        u = self.rng.uniform()
        positive = probs > 0
        totals = np.cumsum(np.where(positive, probs, 0.0))
        hit = np.nonzero(positive & (u < totals))[0]
        if hit.size:
            return int(hit[0])
        return int(np.nonzero(positive)[0][-1])      # rounding left u above the total
