"""Greedy, temperature, top-k, top-p, min-p and penalties, on the host and on the device."""
from .sampler import Rng, Sampler, Sampling, choose_many
