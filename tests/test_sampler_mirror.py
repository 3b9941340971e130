"""The package's host sampler (C++) against the plain sampler of `plain_sampler.py` on random logits
and settings: the same certain tokens, the same probabilities bit for bit (both add in index order
and call the C library's exp), the same draws from the same uniform numbers. No GPU needed.
"""
import math

import numpy as np
import pytest

import plain_gemma2 as P
from kapel_b200.sampling import Sampler, Sampling, choose_many
from plain_sampler import plain_distribution, plain_draw


def random_case(rng):
    n = int(rng.choice([1, 2, 7, 33, 300, 2000]))
    logits = rng.normal(size=n) * float(rng.choice([0.1, 1.0, 8.0]))
    if rng.random() < 0.3:                                   # ties
        logits = np.round(logits, 1)
    if rng.random() < 0.2:
        logits[rng.integers(0, n, size=max(1, n // 5))] = -np.inf
    if rng.random() < 0.08:
        logits[int(rng.integers(n))] = np.nan
    if rng.random() < 0.03:
        logits[:] = -np.inf
    s = Sampling(
        temperature=float(rng.choice([0.0, 0.3, 1.0, 1.7])),
        top_k=None if rng.random() < 0.4 else int(rng.choice([0, 1, 2, 5, 50, n, n + 3])),
        top_p=float(rng.choice([1.0, 0.95, 0.5, 0.1, 0.0])),
        min_p=float(rng.choice([0.0, 0.0, 0.05, 0.5, 1.0])),
        repetition_penalty=float(rng.choice([1.0, 1.0, 1.3, 0.8])),
        frequency_penalty=float(rng.choice([0.0, 0.0, 0.4])),
        presence_penalty=float(rng.choice([0.0, 0.0, 0.25])),
        seed=int(rng.integers(0, 2 ** 40)),
    )
    seq = [int(t) for t in rng.integers(-2, n + 3, size=int(rng.integers(0, 40)))]   # some tokens outside the vocabulary
    return logits, s, seq, int(rng.integers(0, len(seq) + 2))


def plain_of(logits, s, seq, gen_from):
    return plain_distribution(list(logits), s.temperature, s.top_k, s.top_p, s.min_p, s.repetition_penalty,
                              s.frequency_penalty, s.presence_penalty, seq, gen_from)


@pytest.mark.parametrize("seed", range(8))
def test_distributions_and_draws_are_the_plain_ones(seed):
    rng = np.random.default_rng(seed)
    for _ in range(250):
        logits, s, seq, gen_from = random_case(rng)
        want_token, want_probs = plain_of(logits, s, seq, gen_from)
        sampler = Sampler(s)
        token, probs = sampler.distribution(logits, seq, gen_from)
        assert token == want_token, (s, logits[:10])
        if want_probs is None:
            assert probs is None
            assert sampler.choose(logits, seq, gen_from) == want_token
            assert sampler.rng.s == P.PlainRng(s.seed).s                 # a certain choice draws nothing
        else:
            assert probs.tolist() == want_probs                          # bit for bit
            plain_rng = P.PlainRng(s.seed)
            for _ in range(3):
                assert sampler.choose(logits, seq, gen_from) == plain_draw(want_probs, plain_rng.uniform())
            assert sampler.rng.s == plain_rng.s


def test_float32_rows_are_widened_exactly_and_many_requests_choose_as_one_by_one():
    rng = np.random.default_rng(99)
    n, count = 5000, 11
    rows = (rng.normal(size=(count, n)) * 3).astype(np.float32)
    settings = [Sampling(temperature=0.9, top_k=40, seed=i) for i in range(4)]
    settings += [Sampling(temperature=0.7, top_p=0.8, min_p=0.02, seed=20 + i) for i in range(3)]
    settings += [Sampling(repetition_penalty=1.2, presence_penalty=0.1)]              # greedy with penalties
    settings += [Sampling(temperature=1.0, frequency_penalty=0.3, top_k=7, seed=5), Sampling(temperature=1.0, seed=6), Sampling()]
    seqs = [[int(t) for t in rng.integers(0, n, size=60)] for _ in range(count)]
    gen = [int(g) for g in rng.integers(0, 60, size=count)]
    for threads in (1, 3, None):
        many = [Sampler(s) for s in settings]
        single = [Sampler(s) for s in settings]
        for step in range(4):
            got = choose_many(many, rows, seqs, gen, threads=threads)
            want = [single[i].choose(rows[i], seqs[i], gen[i]) for i in range(count)]
            assert got == want
            assert [m.rng.s for m in many] == [s.rng.s for s in single]
    for i in range(count):                                     # and the single ones are the plain ones, from float32
        s = settings[i]
        token, probs = plain_of([float(v) for v in rows[i]], s, seqs[i], gen[i])
        plain_rng = P.PlainRng(s.seed)
        want = token if probs is None else plain_draw(probs, plain_rng.uniform())
        assert Sampler(s).choose(rows[i], seqs[i], gen[i]) == want


def test_top_p_over_many_tokens_needs_more_than_one_batch_of_the_sort():
    n = 3000
    logits = np.zeros(n)                                       # all alike: 0.9 of the mass is 2,700 tokens
    logits[::7] += 1e-9
    s = Sampling(temperature=1.0, top_p=0.9, seed=1)
    _, probs = Sampler(s).distribution(logits, [], 0)
    _, want = plain_of(logits, s, [], 0)
    assert probs.tolist() == want and 2690 < int((probs > 0).sum()) < 2710
    assert math.isclose(float(probs.sum()), 1.0, rel_tol=1e-12)
