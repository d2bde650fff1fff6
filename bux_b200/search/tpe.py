"""Tree-structured Parzen estimator: split the finished trials at the gamma quantile into
good and bad, model each by a Parzen window (Gaussians for numbers, smoothed counts for
choices), and take the candidate drawn from the good model with the best ratio l/g.
`multivariate` scores a candidate by the joint density instead of per-dimension picks."""

from __future__ import annotations

import numpy as np


def _bandwidth(points: np.ndarray) -> float:
    n = max(len(points), 1)
    return max(0.05, 1.06 * (points.std() if n > 1 else 0.25) * n ** -0.2)


def _log_density(q: np.ndarray, points: np.ndarray, categorical: bool, options: int = 0) -> np.ndarray:
    if categorical:
        counts = np.bincount(np.minimum((points * options).astype(int), options - 1), minlength=options) + 1.0
        p = counts / counts.sum()
        return np.log(p[np.minimum((q * options).astype(int), options - 1)])
    pts = np.concatenate([points, [0.5]])       # a wide prior component
    bw = np.concatenate([np.full(len(points), _bandwidth(points)), [0.5]])
    z = (q[:, None] - pts[None, :]) / bw
    dens = np.exp(-0.5 * z * z) / (bw * np.sqrt(2 * np.pi))
    return np.log(dens.mean(1) + 1e-300)


def suggest(x: np.ndarray, y: np.ndarray, dims: int, rng, gamma: float = 0.1, candidates: int = 24,
            multivariate: bool = True, categorical=None, options=None) -> np.ndarray:
    categorical = categorical or [False] * dims
    options = options or [0] * dims
    n_good = max(1, int(np.ceil(gamma * len(y))))
    order = np.argsort(y)
    good, bad = x[order[:n_good]], x[order[n_good:]]
    if len(bad) == 0:
        bad = x
    cand = np.empty((candidates, dims))
    for d in range(dims):
        if categorical[d]:
            counts = np.bincount(np.minimum((good[:, d] * options[d]).astype(int), options[d] - 1),
                                 minlength=options[d]) + 1.0
            pick = rng.choice(options[d], candidates, p=counts / counts.sum())
            cand[:, d] = (pick + 0.5) / options[d]
        else:
            centers = np.concatenate([good[:, d], [0.5]])
            bw = np.concatenate([np.full(len(good), _bandwidth(good[:, d])), [0.5]])
            which = rng.integers(0, len(centers), candidates)
            cand[:, d] = np.clip(rng.normal(centers[which], bw[which]), 0, 1)
    ratio = np.zeros((candidates, dims))
    for d in range(dims):
        ratio[:, d] = (_log_density(cand[:, d], good[:, d], categorical[d], options[d])
                       - _log_density(cand[:, d], bad[:, d], categorical[d], options[d]))
    if multivariate:
        return cand[int(np.argmax(ratio.sum(1)))]
    return np.array([cand[int(np.argmax(ratio[:, d])), d] for d in range(dims)])
