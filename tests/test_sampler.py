"""The host sampler: Kapel's rules (crates/kapel-infer/src/sampling.rs:320-433 tests the same ones)."""
import math

import numpy as np

import plain_gemma2 as P
from kapel_b200.sampling import Rng, Sampler, Sampling


def choose(settings, logits, sequence=(), generated_from=0):
    return Sampler(settings).choose(np.array(logits, dtype=np.float64), list(sequence), generated_from)


def test_generator_is_the_plain_one():
    a, b = Rng(7), P.PlainRng(7)
    assert [a.next_u64() for _ in range(20)] == [b.next_u64() for _ in range(20)]
    assert all(0.0 <= Rng(s).uniform() < 1.0 for s in range(50))
    # SplitMix64 from seed 0: a known first output of the reference algorithm
    assert P.PlainRng(0).s[0] == 0xE220A8397B1DCDAF


def test_greedy_first_max_on_ties_and_no_nan():
    nan = float("nan")
    assert choose(Sampling(), [1.0, 5.0, 5.0, 2.0]) == 1
    assert choose(Sampling(), [nan, -3.0, nan, -3.0]) == 1
    assert choose(Sampling(), [nan, nan]) == 0
    assert Sampling().is_argmax() and not Sampling(repetition_penalty=1.1).is_argmax()
    assert Sampling(temperature=0.7).on_device() and not Sampling(temperature=0.7, top_k=5).on_device()


def test_penalties_come_first():
    logits = [2.0, 1.9, -1.0]
    assert choose(Sampling(repetition_penalty=2.0), logits, [0]) == 1              # 2.0 / 2 < 1.9
    assert choose(Sampling(repetition_penalty=2.0), [-1.0, -1.5, -3.0], [0]) == 1  # -1 * 2 < -1.5
    assert choose(Sampling(frequency_penalty=0.2), logits, [9, 0, 0], generated_from=1) == 1
    assert choose(Sampling(presence_penalty=0.2), logits, [0, 2], generated_from=1) == 0   # prompt tokens do not count
    assert choose(Sampling(presence_penalty=0.2), logits, [2, 0], generated_from=1) == 1


def test_filters_in_order():
    logits = [0.0, math.log(2), math.log(4), math.log(8)]         # probabilities 1/15, 2/15, 4/15, 8/15
    s = Sampler(Sampling(temperature=1.0, top_k=2))
    _, probs = s.distribution(np.array(logits), [], 0)
    assert np.allclose(probs, [0, 0, 1 / 3, 2 / 3])
    _, probs = Sampler(Sampling(temperature=1.0, top_p=0.6)).distribution(np.array(logits), [], 0)
    assert np.allclose(probs, [0, 0, 1 / 3, 2 / 3])                # 8/15 < 0.6 keeps the next one too
    _, probs = Sampler(Sampling(temperature=1.0, top_p=0.5)).distribution(np.array(logits), [], 0)
    assert np.allclose(probs, [0, 0, 0, 1])
    _, probs = Sampler(Sampling(temperature=1.0, min_p=0.3)).distribution(np.array(logits), [], 0)
    assert np.allclose(probs, [0, 0, 1 / 3, 2 / 3])                # floor 0.3 * 8/15 = 0.16
    _, probs = Sampler(Sampling(temperature=0.5)).distribution(np.array(logits), [], 0)
    assert np.allclose(probs, np.array([1, 4, 16, 64]) / 85)
    token, probs = Sampler(Sampling(temperature=1.0)).distribution(np.array([-np.inf, -np.inf]), [], 0)
    assert token == 0 and probs is None


def test_draws_follow_the_probabilities_and_the_seed():
    logits = [0.0, math.log(2), math.log(4)]
    s = Sampler(Sampling(temperature=1.0, seed=3))
    n = 40000
    counts = np.bincount([s.choose(logits) for _ in range(n)], minlength=3) / n
    assert np.abs(counts - np.array([1, 2, 4]) / 7).max() < 0.01
    a = Sampler(Sampling(temperature=1.0, seed=5))
    b = Sampler(Sampling(temperature=1.0, seed=5))
    assert [a.choose(logits) for _ in range(50)] == [b.choose(logits) for _ in range(50)]
    # the plain rule with the same uniform numbers
    r, c = P.PlainRng(9), Sampler(Sampling(temperature=0.8, seed=9))
    lg = list(np.random.default_rng(0).normal(size=30))
    assert [c.choose(lg) for _ in range(100)] == [P.plain_choose(lg, 0.8, r.uniform()) for _ in range(100)]


def test_generation_config_defaults():
    assert Sampling.from_generation_config({}).is_greedy()
    s = Sampling.from_generation_config({"do_sample": True})
    assert (s.temperature, s.top_k, s.top_p) == (1.0, 50, 1.0)
    s = Sampling.from_generation_config({"do_sample": True, "top_k": 0, "temperature": 0.7, "repetition_penalty": 1.2})
    assert (s.temperature, s.top_k, s.repetition_penalty) == (0.7, None, 1.2)
