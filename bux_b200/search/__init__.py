"""Hyperparameter search over the dimensions a `.bux` file writes as distributions.

``methods`` (random / Halton / Sobol points in the unit cube), ``tpe``, ``gp``
(Matérn-5/2 Gaussian process with log-EI / UCB), ``halving`` (ASHA / Hyperband rungs)
and ``search`` (the resumable driver: ``trials.jsonl``, ``best.bux``).
Reference: ``search/search.py``, ``search/gp.py``, ``search/tpe.py``,
``search/halving.py``, ``search/methods.py``, ``search/space.py``.
"""
from .search import Search  # noqa: F401
