"""Gaussian-process Bayesian optimisation: Matérn-5/2 kernel with per-dimension length
scales fitted by marginal likelihood (L-BFGS-B), log expected improvement or a
confidence bound maximised from random and local candidates. Objectives are minimised."""

from __future__ import annotations

import numpy as np
from scipy.linalg import cho_factor, cho_solve
from scipy.optimize import minimize
from scipy.special import erfcx, log1p  # noqa: F401
from scipy.stats import norm


def matern52(a: np.ndarray, b: np.ndarray, scales: np.ndarray) -> np.ndarray:
    d = np.sqrt(np.maximum(((a[:, None, :] - b[None, :, :]) / scales) ** 2, 0).sum(-1))
    r = np.sqrt(5.0) * d
    return (1 + r + r * r / 3) * np.exp(-r)


class GP:
    def __init__(self, x: np.ndarray, y: np.ndarray):
        self.x = np.asarray(x, float)
        y = np.asarray(y, float)
        self.mean, self.std = y.mean(), max(y.std(), 1e-9)
        self.y = (y - self.mean) / self.std
        d = self.x.shape[1]
        theta0 = np.concatenate([np.zeros(d) + np.log(0.5), [np.log(1.0), np.log(1e-2)]])
        bounds = [(np.log(0.05), np.log(5.0))] * d + [(np.log(0.05), np.log(10.0)), (np.log(1e-6), np.log(1.0))]
        best = minimize(self._nll, theta0, method="L-BFGS-B", bounds=bounds)
        self.theta = best.x if np.isfinite(best.fun) else theta0
        self._fit(self.theta)

    def _kernel(self, theta, a, b):
        d = self.x.shape[1]
        return np.exp(theta[d]) * matern52(a, b, np.exp(theta[:d]))

    def _nll(self, theta) -> float:
        d = self.x.shape[1]
        k = self._kernel(theta, self.x, self.x) + (np.exp(theta[d + 1]) + 1e-8) * np.eye(len(self.x))
        try:
            c = cho_factor(k, lower=True)
        except np.linalg.LinAlgError:
            return 1e25
        alpha = cho_solve(c, self.y)
        return float(0.5 * self.y @ alpha + np.log(np.diag(c[0])).sum())

    def _fit(self, theta) -> None:
        d = self.x.shape[1]
        k = self._kernel(theta, self.x, self.x) + (np.exp(theta[d + 1]) + 1e-8) * np.eye(len(self.x))
        self.chol = cho_factor(k, lower=True)
        self.alpha = cho_solve(self.chol, self.y)

    def predict(self, q: np.ndarray):
        """(mean, std) in the objective's units."""
        q = np.atleast_2d(q)
        d = self.x.shape[1]
        ks = self._kernel(self.theta, q, self.x)
        mu = ks @ self.alpha
        v = cho_solve(self.chol, ks.T)
        var = np.maximum(np.exp(self.theta[d]) - (ks * v.T).sum(-1), 1e-12)
        return mu * self.std + self.mean, np.sqrt(var) * self.std


def log_ei(mu, sigma, best) -> np.ndarray:
    """log of the expected improvement below `best`, stable far into the tail."""
    z = (best - mu) / sigma
    out = np.empty_like(z)
    hi = z > -6
    out[hi] = np.log(np.maximum(norm.pdf(z[hi]) + z[hi] * norm.cdf(z[hi]), 1e-300))
    zl = z[~hi]
    # asymptotic: pdf(z)/z^2 for z → -inf
    out[~hi] = norm.logpdf(zl) - 2 * np.log(-zl)
    return out + np.log(sigma)


def suggest(x: np.ndarray, y: np.ndarray, dims: int, rng, acquisition: str = "log_ei", beta: float = 2.0,
            pending: np.ndarray = None, candidates: int = 2048) -> np.ndarray:
    """The next point of the unit cube. `pending` points (running trials) are treated as
    if they had returned the model's mean there (a "believer"), so parallel suggestions differ."""
    gp = GP(x, y)
    if pending is not None and len(pending):
        mu, _ = gp.predict(pending)
        gp = GP(np.vstack([x, pending]), np.concatenate([y, mu]))
    best = float(np.min(y))
    cand = rng.random((candidates, dims))
    top = x[np.argsort(y)[: min(5, len(y))]]
    local = np.clip(top[rng.integers(0, len(top), candidates // 4)] + rng.normal(0, 0.05, (candidates // 4, dims)), 0, 1)
    cand = np.vstack([cand, local])
    mu, sd = gp.predict(cand)
    score = log_ei(mu, sd, best) if acquisition == "log_ei" else -(mu - beta * sd)
    return cand[int(np.argmax(score))]
