"""Points of the unit cube that depend on the trial's index alone: random, Halton, Sobol."""

from __future__ import annotations

import numpy as np

_PRIMES = (2, 3, 5, 7, 11, 13, 17, 19, 23, 29, 31, 37, 41, 43, 47, 53, 59, 61, 67, 71)


def random_point(index: int, dims: int, seed: int) -> np.ndarray:
    return np.random.default_rng((seed, index)).random(dims)


def _radical_inverse(i: int, base: int) -> float:
    x, f = 0.0, 1.0 / base
    while i:
        i, d = divmod(i, base)
        x += d * f
        f /= base
    return x


def halton_point(index: int, dims: int, seed: int) -> np.ndarray:
    """Scrambled by a seeded rotation (Cranley-Patterson), skipping index 0."""
    if dims > len(_PRIMES):
        raise ValueError(f"halton supports up to {len(_PRIMES)} dimensions")
    shift = np.random.default_rng(seed).random(dims)
    raw = np.array([_radical_inverse(index + 1, _PRIMES[d]) for d in range(dims)])
    return (raw + shift) % 1.0


def sobol_point(index: int, dims: int, seed: int) -> np.ndarray:
    from scipy.stats import qmc

    eng = qmc.Sobol(d=dims, scramble=True, seed=seed)
    if index:
        eng.fast_forward(index)
    return eng.random(1)[0]


POINTS = {"random": random_point, "halton": halton_point, "sobol": sobol_point}
